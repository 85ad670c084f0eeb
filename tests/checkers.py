"""The two CPU checkers the tests compare the CUDA library against, as numpy-level functions.

  Oracle        oracle/liboracle.so -- the plain-C restatement (always available; built by `make -C oracle port`)
  ReferenceCpu  oracle/_ref/libminml_cpu_ref.so -- minml's own CPU backend compiled from the reference sources
                (present when it was built in a container that has the reference checkout; it travels as a binary)

Only tests, the smoke check and the benchmark's CPU-baseline leg import this module.
"""
import ctypes
import os
import subprocess

import numpy as np

from minml_b200._abi import mlShape_t, mlTensor_t, DTYPE_FLOAT32

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
ORACLE_DIR = os.path.join(ROOT, "oracle")
ACT = {"linear": 0, "sigmoid": 1, "tanh": 2, "relu": 3, "leaky_relu": 4, "exp": 5}

c_float_p = ctypes.POINTER(ctypes.c_float)
c_i8_p = ctypes.POINTER(ctypes.c_int8)
c_i32_p = ctypes.POINTER(ctypes.c_int32)


def _fp(a):
    return None if a is None else a.ctypes.data_as(c_float_p)


def _i8(a):
    return None if a is None else a.ctypes.data_as(c_i8_p)


def _i32(a):
    return None if a is None else a.ctypes.data_as(c_i32_p)


def _f32(a):
    return None if a is None else np.ascontiguousarray(a, dtype=np.float32)


class Oracle:
    def __init__(self, lib):
        self.lib = lib
        for name in ("oracle_winograd_weight_transform", "oracle_winograd_input_transform", "oracle_winograd_output_transform", "oracle_gemm",
                     "oracle_gemm_i8_nt", "oracle_conv2d", "oracle_conv2d_int8", "oracle_quantize_weights", "oracle_scale_shift_act",
                     "oracle_im2row", "oracle_global_average_pooling", "oracle_layernorm", "oracle_mha_forward", "oracle_unpack_input",
                     "oracle_softmax", "oracle_add_bias_act"):
            getattr(lib, name).restype = None

    def winograd_weight_transform(self, w, tile=4, invert=False):
        w = _f32(w)
        cout, k, _, cin = w.shape
        p = tile + k - 1
        u = np.empty((p * p, cout, cin), np.float32)
        self.lib.oracle_winograd_weight_transform(tile, k, _fp(w), _fp(u), cout, cin, int(invert))
        return u

    def winograd_input_transform(self, x, tile=4, k=3):
        x = _f32(x)
        b, h, w, c = x.shape
        p = tile + k - 1
        tiles = b * ((h + tile - 1) // tile) * ((w + tile - 1) // tile)
        v = np.empty((p * p, tiles, c), np.float32)
        self.lib.oracle_winograd_input_transform(tile, k, _fp(x), _fp(v), b, h, w, c)
        return v

    def winograd_gradient_transform(self, dy, tile=4, k=3):
        dy = _f32(dy)
        b, h, w, c = dy.shape
        p = tile + k - 1
        tiles = b * ((h + tile - 1) // tile) * ((w + tile - 1) // tile)
        m = np.empty((p * p, tiles, c), np.float32)
        self.lib.oracle_winograd_gradient_transform(tile, k, _fp(dy), _fp(m), b, h, w, c)
        return m

    def winograd_update_transform(self, m, tile=4, k=3):
        m = _f32(m)
        _, cout, cin = m.shape
        dw = np.empty((cout, k, k, cin), np.float32)
        self.lib.oracle_winograd_update_transform(tile, k, _fp(m), _fp(dw), cout, cin)
        return dw

    def act_bias_copy_backward(self, dy, y, dx=None, db=None, beta_dx=0.0, beta_db=0.0, act="linear", with_dx=True, with_db=True):
        """Returns (dy after the activation derivative, dx or None, db or None)."""
        dy, y = _f32(dy).copy(), _f32(y)
        c = dy.shape[-1]
        dx_out = (np.zeros_like(dy) if dx is None else _f32(dx).copy()) if with_dx else None
        db_out = (np.zeros(c, np.float32) if db is None else _f32(db).copy()) if with_db else None
        self.lib.oracle_act_bias_copy_backward(_fp(dy), _fp(y), _fp(dx_out), _fp(db_out), ctypes.c_float(beta_dx), ctypes.c_float(beta_db), ACT[act],
                                               ctypes.c_size_t(dy.size // c), c)
        return dy, dx_out, db_out

    def winograd_output_transform(self, m, out_shape, bias=None, ext=None, act="linear", tile=4, k=3):
        m, bias, ext = _f32(m), _f32(bias), _f32(ext)
        b, h, w, c = out_shape
        y = np.empty(out_shape, np.float32)
        self.lib.oracle_winograd_output_transform(tile, k, _fp(m), _fp(y), _fp(bias), _fp(ext), ACT[act], b, h, w, c)
        return y

    def gemm(self, op_a, a, op_b, b, c=None, alpha=1.0, beta=0.0):
        a, b = _f32(a), _f32(b)
        ta, tb = op_a == "t", op_b == "t"
        rows = a.shape[1] if ta else a.shape[0]
        cols = b.shape[0] if tb else b.shape[1]
        k = b.shape[1] if tb else b.shape[0]
        out = np.zeros((rows, cols), np.float32) if c is None else _f32(c).copy()
        self.lib.oracle_gemm(int(ta), int(tb), rows, cols, k, ctypes.c_float(alpha), _fp(a), a.shape[1], _fp(b), b.shape[1], ctypes.c_float(beta),
                             _fp(out), cols)
        return out

    def gemm_i8_nt(self, a, b):
        a, b = np.ascontiguousarray(a, np.int8), np.ascontiguousarray(b, np.int8)
        c = np.empty((a.shape[0], b.shape[0]), np.int32)
        self.lib.oracle_gemm_i8_nt(a.shape[0], b.shape[0], a.shape[1], _i8(a), _i8(b), _i32(c))
        return c

    def conv2d(self, x, w, bias=None, ext=None, act="linear"):
        x, w, bias, ext = _f32(x), _f32(w), _f32(bias), _f32(ext)
        b, h, wd, cin = x.shape
        cout, k = w.shape[0], w.shape[1]
        y = np.empty((b, h, wd, cout), np.float32)
        self.lib.oracle_conv2d(_fp(x), _fp(w), _fp(bias), _fp(ext), _fp(y), ACT[act], b, h, wd, cin, cout, k)
        return y

    def conv2d_int8(self, x, w, channel_scales, bias, input_zero, out_qd=(1.0, 0.0), act="linear", ext=None, ext_qd=(1.0, 0.0)):
        """Returns (y_int8, y_fp32, acc_int32)."""
        x, w = np.ascontiguousarray(x, np.int8), np.ascontiguousarray(w, np.int8)
        ext = None if ext is None else np.ascontiguousarray(ext, np.int8)
        channel_scales, bias = _f32(channel_scales), _f32(bias)
        b, h, wd, cin = x.shape
        cout, k = w.shape[0], w.shape[1]
        y8 = np.empty((b, h, wd, cout), np.int8)
        yf = np.empty((b, h, wd, cout), np.float32)
        acc = np.empty((b, h, wd, cout), np.int32)
        self.lib.oracle_conv2d_int8(_i8(x), _i8(w), _fp(channel_scales), _fp(bias), _i8(ext), ctypes.c_float(ext_qd[0]), ctypes.c_float(ext_qd[1]),
                                    int(input_zero), ctypes.c_float(out_qd[0]), ctypes.c_float(out_qd[1]), ACT[act], _i8(y8), _fp(yf), _i32(acc),
                                    b, h, wd, cin, cout, k)
        return y8, yf, acc

    def quantize_weights(self, w, bias, in_scale, in_shift):
        w, bias = _f32(w), _f32(bias)
        cout = w.shape[0]
        per = int(np.prod(w.shape[1:]))
        q = np.empty(w.shape, np.int8)
        cs = np.empty(cout, np.float32)
        qb = np.empty(cout, np.float32)
        self.lib.oracle_quantize_weights(_fp(w), _fp(bias), ctypes.c_float(in_scale), ctypes.c_float(in_shift), _i8(q), _fp(cs), _fp(qb), cout, per)
        return q, cs, qb

    def scale_shift_act(self, acc, scales, bias, out_qd=(1.0, 0.0), act="linear", ext=None, ext_qd=(1.0, 0.0)):
        acc = np.ascontiguousarray(acc, np.int32)
        ext = None if ext is None else np.ascontiguousarray(ext, np.int8)
        channels = acc.shape[-1]
        rows = acc.size // channels
        y8 = np.empty(acc.shape, np.int8)
        yf = np.empty(acc.shape, np.float32)
        self.lib.oracle_scale_shift_act(_i32(acc), _fp(_f32(scales)), _fp(_f32(bias)), _i8(ext), ctypes.c_float(ext_qd[0]), ctypes.c_float(ext_qd[1]),
                                        ctypes.c_float(out_qd[0]), ctypes.c_float(out_qd[1]), ACT[act], _i8(y8), _fp(yf), ctypes.c_size_t(rows),
                                        channels)
        return y8, yf

    def im2row(self, x, k, invert=False, pad=None):
        x = np.ascontiguousarray(x)
        b, h, w, c = x.shape
        out = np.empty((b * h * w, k * k * c), x.dtype)
        pad_arr = None if pad is None else np.asarray([pad], dtype=x.dtype)
        self.lib.oracle_im2row(x.ctypes.data_as(ctypes.c_void_p), out.ctypes.data_as(ctypes.c_void_p), b, h, w, c, k, int(invert), x.itemsize,
                               None if pad_arr is None else pad_arr.ctypes.data_as(ctypes.c_void_p))
        return out

    def batchnorm_inference(self, x, gamma, beta_bn, avg_var, act="linear", alpha=1.0, beta=0.0, y=None):
        x = _f32(x)
        c = x.shape[-1]
        out = np.zeros_like(x) if y is None else _f32(y).copy()
        self.lib.oracle_batchnorm_inference(_fp(x), _fp(out), _fp(_f32(gamma)), _fp(_f32(beta_bn)), _fp(_f32(avg_var)), ctypes.c_float(alpha),
                                            ctypes.c_float(beta), ACT[act], ctypes.c_size_t(x.size // c), c)
        return out

    def fold_batchnorm(self, weights, bias, gamma, beta_bn, avg_var):
        """Returns (folded weights, folded bias); [k, k, c] weights are depthwise (one channel per column)."""
        w, b = _f32(weights).copy(), _f32(bias).copy()
        per_row = w.ndim != 3
        outer = w.shape[0] if per_row else w.shape[0] * w.shape[1]
        self.lib.oracle_fold_batchnorm(_fp(w), _fp(b), _fp(_f32(gamma)), _fp(_f32(beta_bn)), _fp(_f32(avg_var)), outer, w.size // outer, int(per_row))
        return w, b

    def depthwise_conv(self, x, w, bias=None, alpha=1.0, beta=0.0, y=None):
        x, w = _f32(x), _f32(w)
        b, h, wd, c = x.shape
        out = np.zeros_like(x) if y is None else _f32(y).copy()
        self.lib.oracle_depthwise_conv(_fp(x), _fp(w), _fp(_f32(bias)), _fp(out), ctypes.c_float(alpha), ctypes.c_float(beta), b, h, wd, c, w.shape[0])
        return out

    def depthwise_conv_int8(self, x, w, scales, bias, out_qd=(1.0, 0.0), input_zero=0):
        """Returns (y_int8, y_fp32)."""
        x, w = np.ascontiguousarray(x, np.int8), np.ascontiguousarray(w, np.int8)
        b, h, wd, c = x.shape
        y8, yf = np.empty(x.shape, np.int8), np.empty(x.shape, np.float32)
        self.lib.oracle_depthwise_conv_int8(_i8(x), _i8(w), _fp(_f32(scales)), _fp(_f32(bias)), _i8(y8), _fp(yf), ctypes.c_float(out_qd[0]),
                                            ctypes.c_float(out_qd[1]), int(input_zero), b, h, wd, c, w.shape[0])
        return y8, yf

    def channel_scaling(self, x, scales, alpha=1.0, beta=0.0, y=None):
        x = _f32(x)
        b, c = x.shape[0], x.shape[-1]
        out = np.zeros_like(x) if y is None else _f32(y).copy()
        self.lib.oracle_channel_scaling(_fp(x), _fp(_f32(scales)), _fp(out), ctypes.c_float(alpha), ctypes.c_float(beta), b, x.size // (b * c), c)
        return out

    def rmsnorm(self, x, gamma=None):
        x = _f32(x)
        y = np.empty_like(x)
        c = x.shape[-1]
        self.lib.oracle_rmsnorm(_fp(x), _fp(y), _fp(_f32(gamma)), ctypes.c_size_t(x.size // c), c)
        return y

    def space_to_depth(self, x, out_hw):
        """x [b, h, w, c] of any dtype -> [b, oh, ow, p*q*c]; raises when the shapes do not fit."""
        x = np.ascontiguousarray(x)
        b, h, w, c = x.shape
        oh, ow = out_hw
        p, q = -(-h // oh), -(-w // ow)
        y = np.empty((b, oh, ow, p * q * c), x.dtype)
        self.lib.oracle_space_to_depth.restype = ctypes.c_int
        ok = self.lib.oracle_space_to_depth(ctypes.c_void_p(x.ctypes.data), ctypes.c_void_p(y.ctypes.data), x.dtype.itemsize, b, h, w, c, oh, ow)
        if not ok or y.shape[3] != p * q * c:
            raise ValueError("shapes do not fit")
        return y

    def depth_to_space(self, x, out_hw, fill=0):
        """x [b, ih, iw, p*q*c] -> [b, h, w, c]."""
        x = np.ascontiguousarray(x)
        b, ih, iw, deep = x.shape
        h, w = out_hw
        p, q = -(-h // ih), -(-w // iw)
        y = np.full((b, h, w, deep // (p * q)), fill, x.dtype)
        self.lib.oracle_depth_to_space.restype = ctypes.c_int
        if not self.lib.oracle_depth_to_space(ctypes.c_void_p(x.ctypes.data), ctypes.c_void_p(y.ctypes.data), x.dtype.itemsize, b, ih, iw, h, w,
                                              y.shape[3]):
            raise ValueError("shapes do not fit")
        return y

    def global_average_pooling(self, x, alpha=1.0, beta=0.0, y=None):
        x = _f32(x)
        b, h, w, c = x.shape
        out = np.zeros((b, c), np.float32) if y is None else _f32(y).copy()
        self.lib.oracle_global_average_pooling(_fp(x), _fp(out), ctypes.c_float(alpha), ctypes.c_float(beta), b, h * w, c)
        return out

    def layernorm(self, x, gamma, beta, ext=None):
        x = _f32(x)
        y = np.empty_like(x)
        c = x.shape[-1]
        self.lib.oracle_layernorm(_fp(x), _fp(y), _fp(_f32(gamma)), _fp(_f32(beta)), _fp(_f32(ext)), ctypes.c_size_t(x.size // c), c)
        return y

    def mha_forward(self, x, heads, table=None, symmetric=False):
        x, table = _f32(x), _f32(table)
        b, h, w, ch = x.shape
        parts = 2 if symmetric else 3
        d = ch // (parts * heads)
        y = np.empty((b, h, w, heads * d), np.float32)
        self.lib.oracle_mha_forward(_fp(x), _fp(y), _fp(table), b, h, w, heads, d, int(symmetric), 0 if table is None else table.shape[1])
        return y

    def unpack_input(self, packed, shape):
        packed = np.ascontiguousarray(packed, np.uint32)
        y = np.empty(shape, np.float32)
        c = shape[-1]
        self.lib.oracle_unpack_input(packed.ctypes.data_as(ctypes.c_void_p), _fp(y), ctypes.c_size_t(y.size // c), c)
        return y

    def softmax(self, x):
        x = _f32(x)
        y = np.empty_like(x)
        c = x.shape[-1]
        self.lib.oracle_softmax(_fp(x), _fp(y), ctypes.c_size_t(x.size // c), c)
        return y

    def add_bias_act(self, x, bias, act="linear"):
        x = _f32(x)
        y = np.empty_like(x)
        c = x.shape[-1]
        self.lib.oracle_add_bias_act(_fp(x), _fp(_f32(bias)), _fp(y), ACT[act], ctypes.c_size_t(x.size // c), c)
        return y


def load_oracle():
    path = os.path.join(ORACLE_DIR, "liboracle.so")
    src = os.path.join(ORACLE_DIR, "oracle.c")
    if not os.path.exists(path) or os.path.getmtime(path) < os.path.getmtime(src):
        subprocess.run(["make", "-C", ORACLE_DIR, "port"], check=True, capture_output=True)
    return Oracle(ctypes.CDLL(path))


# ------------------------------------------------------------------------------------------------ reference CPU backend
def _shape(dims):
    s = mlShape_t()
    s.rank = len(dims)
    for i, d in enumerate(dims):
        s.dim[i] = int(d)
    return s


def _tensor(a):
    t = mlTensor_t()
    if a is None:
        t.data, t.dtype, t.rank = None, 0, 0
        return t
    t.data = a.ctypes.data
    t.dtype = DTYPE_FLOAT32
    t.rank = a.ndim
    for i, d in enumerate(a.shape):
        t.dim[i] = int(d)
    return t


def _vp(a):
    return None if a is None else ctypes.c_void_p(a.ctypes.data)


class ReferenceCpu:
    """fp32 calls into minml's CPU backend through its own C ABI (include/minml/backend/cpu_backend.h)."""

    def __init__(self, lib):
        self.lib = lib
        lib.cpu_create_context.restype = ctypes.c_void_p
        self.ctx = ctypes.c_void_p(lib.cpu_create_context())
        S, V, I, F, B, C = mlShape_t, ctypes.c_void_p, ctypes.c_int, ctypes.c_float, ctypes.c_bool, ctypes.c_char
        T = mlTensor_t
        sigs = {
            "cpu_winograd_weight_transform": [V, I, I, S, V, V, B],
            "cpu_winograd_input_transform": [V, I, I, S, S, V, V],
            "cpu_winograd_output_transform": [V, I, I, S, S, V, V, V, V, I],
            "cpu_winograd_gradient_transform": [V, I, I, S, S, V, V],
            "cpu_winograd_update_transform": [V, I, I, S, V, V],
            "cpu_gemm": [V, I, S, V, S, V, S, V, C, C, F, F],
            "cpu_gemm_batched": [V, I, S, V, S, V, S, V, C, C, F, F],
            "cpu_gemm_ex": [V, I, S, V, F, C, S, V, C, S, V, F, S, V, V, I],
            "cpu_add_bias_act": [V, I, S, V, V, V, I],
            "cpu_im2row": [V, I, S, V, V, I, B, V],
            "cpu_global_average_pooling_forward": [V, F, T, F, T],
            "cpu_layernorm_forward": [V, S, I, V, V, V, V, V],
            "cpu_multi_head_attention_forward": [V, T, T, T, T, T, I],
            "cpu_unpack_input": [V, S, I, V, V],
            "cpu_activation_forward": [V, I, S, V, V, I],
            "cpu_batchnorm_inference": [V, I, S, V, V, V, I],
            "cpu_fold_batchnorm": [V, T, T, T, T, T],
            "cpu_depthwise_conv_forward": [V, F, T, T, T, F, T],
            "cpu_channel_scaling_forward": [V, F, T, T, F, T],
            "cpu_rmsnorm_forward": [V, S, I, V, V, V],
            "cpu_space_to_depth": [V, I, S, V, S, V],
            "cpu_depth_to_space": [V, I, S, V, S, V],
        }
        for name, argtypes in sigs.items():
            fn = getattr(lib, name)
            fn.argtypes = argtypes
            fn.restype = None
        lib.cpu_multi_head_attention_get_workspace_size.argtypes = [S, S, I, B]
        lib.cpu_multi_head_attention_get_workspace_size.restype = I

    def winograd_weight_transform(self, w, tile=4, invert=False):
        w = _f32(w)
        cout, k, _, cin = w.shape
        p = tile + k - 1
        u = np.zeros((p * p, cout, cin), np.float32)
        self.lib.cpu_winograd_weight_transform(self.ctx, tile, DTYPE_FLOAT32, _shape(w.shape), _vp(w), _vp(u), bool(invert))
        return u

    def winograd_input_transform(self, x, weight_shape, tile=4):
        x = _f32(x)
        b, h, w, c = x.shape
        p = tile + weight_shape[1] - 1
        tiles = b * ((h + tile - 1) // tile) * ((w + tile - 1) // tile)
        v = np.zeros((p * p, tiles, c), np.float32)
        self.lib.cpu_winograd_input_transform(self.ctx, tile, DTYPE_FLOAT32, _shape(weight_shape), _shape(x.shape), _vp(x), _vp(v))
        return v

    def winograd_gradient_transform(self, dy, weight_shape, tile=4):
        dy = _f32(dy)
        b, h, w, c = dy.shape
        p = tile + weight_shape[1] - 1
        tiles = b * ((h + tile - 1) // tile) * ((w + tile - 1) // tile)
        m = np.zeros((p * p, tiles, c), np.float32)
        self.lib.cpu_winograd_gradient_transform(self.ctx, tile, DTYPE_FLOAT32, _shape(weight_shape), _shape(dy.shape), _vp(dy), _vp(m))
        return m

    def winograd_update_transform(self, m, weight_shape, tile=4):
        m = _f32(m)
        dw = np.zeros(weight_shape, np.float32)
        self.lib.cpu_winograd_update_transform(self.ctx, tile, DTYPE_FLOAT32, _shape(weight_shape), _vp(m), _vp(dw))
        return dw

    def winograd_output_transform(self, m, weight_shape, out_shape, bias=None, ext=None, act="linear", tile=4):
        m, bias, ext = _f32(m), _f32(bias), _f32(ext)
        y = np.zeros(out_shape, np.float32)
        self.lib.cpu_winograd_output_transform(self.ctx, tile, DTYPE_FLOAT32, _shape(weight_shape), _shape(out_shape), _vp(m), _vp(y), _vp(bias),
                                               _vp(ext), ACT[act])
        return y

    def gemm(self, op_a, a, op_b, b, c=None, alpha=1.0, beta=0.0, batched=False):
        a, b = _f32(a), _f32(b)
        ta, tb = op_a == "t", op_b == "t"
        rows = a.shape[-1] if ta else a.shape[-2]
        cols = b.shape[-2] if tb else b.shape[-1]
        shape = ((a.shape[0],) if batched else ()) + (rows, cols)
        out = np.zeros(shape, np.float32) if c is None else _f32(c).copy()
        fn = self.lib.cpu_gemm_batched if batched else self.lib.cpu_gemm
        fn(self.ctx, DTYPE_FLOAT32, _shape(out.shape), _vp(out), _shape(a.shape), _vp(a), _shape(b.shape), _vp(b), op_a.encode(), op_b.encode(),
           alpha, beta)
        return out

    def gemm_ex(self, a, b, bias=None, act="linear", alpha=1.0, beta=0.0, c=None):
        """D = act(alpha * A B^T + beta * C + bias)"""
        a, b, bias, c = _f32(a), _f32(b), _f32(bias), _f32(c)
        d = np.zeros((a.shape[0], b.shape[0]), np.float32)
        cc = c if c is not None else d
        self.lib.cpu_gemm_ex(self.ctx, DTYPE_FLOAT32, _shape(d.shape), _vp(d), alpha, b"n", _shape(a.shape), _vp(a), b"t", _shape(b.shape), _vp(b),
                             beta, _shape(cc.shape), _vp(cc), _vp(bias), ACT[act])
        return d

    def conv3x3_winograd(self, x, w, bias=None, ext=None, act="linear", tile=4, u=None):
        """The reference's own three-step 3x3 convolution (src/layers/Conv2D.cpp:365-377) on its CPU backend."""
        x, w = _f32(x), _f32(w)
        if u is None:
            u = self.winograd_weight_transform(w, tile)
        v = self.winograd_input_transform(x, w.shape, tile)
        m = self.gemm("n", v, "t", u, batched=True)
        out_shape = x.shape[:3] + (w.shape[0],)
        return self.winograd_output_transform(m, w.shape, out_shape, bias, ext, act, tile)

    def batchnorm_inference(self, x, gamma, beta_bn, avg_var, act="linear"):
        """cpu_batchnorm_inference takes one [4, c] fp32 tensor: mean, variance, gamma, beta (src/backend/cpu/normalization.cpp:134-139)."""
        x = _f32(x)
        c = x.shape[-1]
        packed = np.ascontiguousarray(np.concatenate([_f32(avg_var).reshape(2, c), _f32(gamma).reshape(1, c), _f32(beta_bn).reshape(1, c)]), np.float32)
        y = np.zeros_like(x)
        self.lib.cpu_batchnorm_inference(self.ctx, DTYPE_FLOAT32, _shape(x.shape), _vp(x), _vp(y), _vp(packed), ACT[act])
        return y

    def fold_batchnorm(self, weights, bias, gamma, beta_bn, avg_var):
        w, b = _f32(weights).copy(), _f32(bias).copy()
        g, bb, av = _f32(gamma), _f32(beta_bn), _f32(avg_var)
        self.lib.cpu_fold_batchnorm(self.ctx, _tensor(w), _tensor(b), _tensor(g), _tensor(bb), _tensor(av))
        return w, b

    def depthwise_conv(self, x, w, bias):
        x, w, bias = _f32(x), _f32(w), _f32(bias)
        y = np.zeros_like(x)
        self.lib.cpu_depthwise_conv_forward(self.ctx, 1.0, _tensor(x), _tensor(w), _tensor(bias), 0.0, _tensor(y))
        return y

    def channel_scaling(self, x, scales):
        x, scales = _f32(x), _f32(scales)
        y = np.zeros_like(x)
        self.lib.cpu_channel_scaling_forward(self.ctx, 1.0, _tensor(x), _tensor(scales), 0.0, _tensor(y))
        return y

    def global_average_pooling(self, x):
        x = _f32(x)
        y = np.zeros((x.shape[0], x.shape[3]), np.float32)
        self.lib.cpu_global_average_pooling_forward(self.ctx, 1.0, _tensor(x), 0.0, _tensor(y))
        return y

    def rmsnorm(self, x, gamma=None):
        x = _f32(x)
        y = np.zeros_like(x)
        self.lib.cpu_rmsnorm_forward(self.ctx, _shape(x.shape), DTYPE_FLOAT32, _vp(x), _vp(y), _vp(_f32(gamma)))
        return y

    def space_to_depth(self, x, out_shape):
        x = _f32(x)
        y = np.full(out_shape, np.nan, np.float32)
        self.lib.cpu_space_to_depth(self.ctx, DTYPE_FLOAT32, _shape(x.shape), _vp(x), _shape(out_shape), _vp(y))
        return y

    def depth_to_space(self, x, out_shape):
        x = _f32(x)
        y = np.zeros(out_shape, np.float32)
        self.lib.cpu_depth_to_space(self.ctx, DTYPE_FLOAT32, _shape(x.shape), _vp(x), _shape(out_shape), _vp(y))
        return y

    def layernorm(self, x, gamma, beta, ext=None):
        x = _f32(x)
        y = np.zeros_like(x)
        self.lib.cpu_layernorm_forward(self.ctx, _shape(x.shape), DTYPE_FLOAT32, _vp(x), _vp(y), _vp(_f32(gamma)), _vp(_f32(beta)), _vp(_f32(ext)))
        return y

    def mha_forward(self, x, heads, table=None):
        x, table = _f32(x), _f32(table)
        b, h, w, ch = x.shape
        d = ch // (3 * heads)
        y = np.zeros((b, h, w, heads * d), np.float32)
        ws = np.zeros(b * heads * (h * w) ** 2 + 1024, np.float32)
        self.lib.cpu_multi_head_attention_forward(self.ctx, _tensor(x), _tensor(y), _tensor(table), _tensor(ws), _tensor(None), heads)
        return y

    def unpack_input(self, packed, shape):
        packed = np.ascontiguousarray(packed, np.uint32)
        y = np.zeros(shape, np.float32)
        self.lib.cpu_unpack_input(self.ctx, _shape(shape), DTYPE_FLOAT32, _vp(y), _vp(packed))
        return y

    def add_bias_act(self, x, bias, act="linear"):
        x, bias = _f32(x), _f32(bias)
        y = np.zeros_like(x)
        self.lib.cpu_add_bias_act(self.ctx, DTYPE_FLOAT32, _shape(x.shape), _vp(y), _vp(x), _vp(bias), ACT[act])
        return y

    def im2row(self, x, k, invert=False):
        x = _f32(x)
        b, h, w, c = x.shape
        out = np.zeros((b * h * w, k * k * c), np.float32)
        self.lib.cpu_im2row(self.ctx, DTYPE_FLOAT32, _shape(x.shape), _vp(out), _vp(x), k, bool(invert), None)
        return out


def load_reference_cpu():
    path = os.path.join(ORACLE_DIR, "_ref", "libminml_cpu_ref.so")
    if not os.path.exists(path):
        return None
    return ReferenceCpu(ctypes.CDLL(path))
