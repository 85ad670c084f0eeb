"""Seeded synthetic weights and inputs of the benchmark configurations (numpy only).

The author's own networks and positions are private, so every configuration is measured and checked on stand-ins with the
stated shapes and value distributions: Bernoulli(0.3) feature planes, He-normal convolution weights, N(0, 0.01) biases,
N(0, 0.02) weights for the conv + attention block.  The same arrays feed the GPU run and the CPU checkers.  This module
imports neither torch nor the CUDA library, so a process that only times a CPU implementation never maps them.
"""
import numpy as np


def he_normal(rng, shape, fan_in):
    return (rng.standard_normal(shape) * np.sqrt(2.0 / fan_in)).astype(np.float32)


def make_trunk_weights(seed, in_planes, channels, blocks):
    """He-normal weights, N(0, 0.01) biases; the same arrays feed the GPU run and the CPU checkers."""
    rng = np.random.default_rng(seed)
    w = {"stem_w": he_normal(rng, (channels, 3, 3, in_planes), 9 * in_planes), "stem_b": (rng.standard_normal(channels) * 0.01).astype(np.float32)}
    for i in range(blocks):
        for j in (1, 2):
            w["b%d_w%d" % (i, j)] = he_normal(rng, (channels, 3, 3, channels), 9 * channels)
            w["b%d_b%d" % (i, j)] = (rng.standard_normal(channels) * 0.01).astype(np.float32)
    w["policy_w"] = he_normal(rng, (1, 1, 1, channels), channels)
    w["policy_b"] = (rng.standard_normal(1) * 0.01).astype(np.float32)
    w["value_w"] = he_normal(rng, (3, channels), channels)
    w["value_b"] = (rng.standard_normal(3) * 0.01).astype(np.float32)
    return w


def make_hybrid_weights(seed, embed, heads, ffn, board):
    """N(0, 0.02) weights for the conv + attention block: a 3x3 residual block, pre-LN attention with a relative-position
    table [heads, 2R-1, round_up(2R-1, 4)] (R = board size), and a ReLU feed-forward network embed -> ffn -> embed."""
    rng = np.random.default_rng(seed)

    def n(*shape):
        return (rng.standard_normal(shape) * 0.02).astype(np.float32)
    size = 2 * board - 1
    return {
        "c1_w": n(embed, 3, 3, embed), "c1_b": n(embed), "c2_w": n(embed, 3, 3, embed), "c2_b": n(embed),
        "ln1_g": np.ones(embed, np.float32), "ln1_b": np.zeros(embed, np.float32),
        "qkv_w": n(3 * embed, 1, 1, embed), "qkv_b": n(3 * embed), "table": n(heads, size, (size + 3) // 4 * 4),
        "proj_w": n(embed, 1, 1, embed), "proj_b": n(embed),
        "ln2_g": np.ones(embed, np.float32), "ln2_b": np.zeros(embed, np.float32),
        "ffn1_w": n(ffn, 1, 1, embed), "ffn1_b": n(ffn), "ffn2_w": n(embed, 1, 1, ffn), "ffn2_b": n(embed),
    }


def pack_planes(x01):
    """[..., c] array of {0, 1} -> uint32 words [..., ceil(c / 32)], channel j in bit j % 32 of word j // 32 (the layout
    cuda_unpack_input reads, src/backend/cuda/kernels/conversion.cu:38-45)."""
    c = x01.shape[-1]
    words = (c + 31) // 32
    out = np.zeros(x01.shape[:-1] + (words,), np.uint32)
    for j in range(c):
        out[..., j // 32] |= (x01[..., j].astype(np.uint32) & 1) << np.uint32(j % 32)
    return out


def bernoulli_planes(shape, seed, p=0.3):
    """({0, 1} planes as fp32 [b, h, w, planes], the same bit-packed as int32 words)."""
    x = (np.random.default_rng(seed).random(shape) < p).astype(np.float32)
    return x, pack_planes(x).view(np.int32)
