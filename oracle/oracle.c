/*
 * oracle.c -- TEST INFRASTRUCTURE, NOT PRODUCT CODE.
 *
 * A plain-C restatement of the arithmetic that minml's CPU backend performs on the convolution / matrix-multiply
 * inference path.  It exists so the CUDA library can be checked against an independent implementation; only the
 * test-suite, the smoke check and the benchmark's CPU-baseline leg may load it.  The library never calls it.
 *
 * Pinned against: the known-answer vectors of the reference's test/backend/test_winograd.cpp:218-394 (transcribed in
 * tests/golden/winograd_known_answers.json) and, where the reference checkout is available, against the reference's
 * own CPU backend compiled from source (oracle/_ref/libminml_cpu_ref.so) -- see tests/test_oracle.py.
 *
 * Conventions: NHWC dense tensors, fp32 data, double accumulation for sums of products (so the oracle is the more
 * accurate side of every comparison); integer paths are exact.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

enum { ACT_LINEAR, ACT_SIGMOID, ACT_TANH, ACT_RELU, ACT_LEAKY_RELU, ACT_EXP };

static float activate(float x, int act)
{ /* reference: src/backend/cpu/kernels/def_kernels.cpp activation set; leaky slope 0.1 */
	switch (act)
	{
		case ACT_SIGMOID: return 1.0f / (1.0f + expf(-x));
		case ACT_TANH: return tanhf(x);
		case ACT_RELU: return x > 0.0f ? x : 0.0f;
		case ACT_LEAKY_RELU: return x > 0.0f ? x : 0.1f * x;
		case ACT_EXP: return expf(x);
		default: return x;
	}
}

/* ---------------------------------------------------------------------------------------------------------------
 * Winograd transform matrices.  Reference: src/backend/cpu/winograd/def_winograd_kernels.cpp:87-378 and the explicit
 * matrices of test/backend/test_winograd.cpp:62-213.  Interpolation points 0, +-1, +-2, infinity.
 * ------------------------------------------------------------------------------------------------------------- */
static const double BT_6[6][6] = {
	{ 1.0, 0.0, -1.25, 0.0, 0.25, 0.0 },
	{ 0.0, 1.0, 1.0, -0.25, -0.25, 0.0 },
	{ 0.0, -1.0, 1.0, 0.25, -0.25, 0.0 },
	{ 0.0, -1.0, -0.5, 1.0, 0.5, 0.0 },
	{ 0.0, 1.0, -0.5, -1.0, 0.5, 0.0 },
	{ 0.0, 1.0, 0.0, -1.25, 0.0, 0.25 } };
static const double BT_4[4][4] = { { 1, 0, -1, 0 }, { 0, 1, 1, 0 }, { 0, -1, 1, 0 }, { 0, -1, 0, 1 } };
static const double G_43[6][3] = {
	{ 1.0, 0.0, 0.0 },
	{ 2.0 / 3, 2.0 / 3, 2.0 / 3 },
	{ 2.0 / 3, -2.0 / 3, 2.0 / 3 },
	{ 1.0 / 3, 2.0 / 3, 4.0 / 3 },
	{ 1.0 / 3, -2.0 / 3, 4.0 / 3 },
	{ 0.0, 0.0, 2.0 } };
static const double G_23[4][3] = { { 1, 0, 0 }, { 0.5, 0.5, 0.5 }, { 0.5, -0.5, 0.5 }, { 0, 0, 1 } };
static const double G_25[6][5] = {
	{ 1, 0, 0, 0, 0 },
	{ 2.0 / 3, 2.0 / 3, 2.0 / 3, 2.0 / 3, 2.0 / 3 },
	{ 2.0 / 3, -2.0 / 3, 2.0 / 3, -2.0 / 3, 2.0 / 3 },
	{ 1.0 / 6, 2.0 / 6, 4.0 / 6, 8.0 / 6, 16.0 / 6 },
	{ 1.0 / 6, -2.0 / 6, 4.0 / 6, -8.0 / 6, 16.0 / 6 },
	{ 0, 0, 0, 0, 2 } };
static const double AT_43[4][6] = {
	{ 1, 1, 1, 0.25, 0.25, 0 },
	{ 0, 1, -1, 0.5, -0.5, 0 },
	{ 0, 1, 1, 1, 1, 0 },
	{ 0, 1, -1, 2, -2, 2 } };
static const double AT_23[2][4] = { { 1, 1, 1, 0 }, { 0, 1, -1, 1 } };
static const double AT_25[2][6] = { { 1, 1, 1, 0.5, 0.5, 0 }, { 0, 1, -1, 1, -1, 2 } };

static double bt_at(int p, int r, int c) { return p == 6 ? BT_6[r][c] : BT_4[r][c]; }
static double g_at(int tile, int k, int r, int c) { return k == 5 ? G_25[r][c] : (tile == 4 ? G_43[r][c] : G_23[r][c]); }
static double at_at(int tile, int k, int r, int c) { return k == 5 ? AT_25[r][c] : (tile == 4 ? AT_43[r][c] : AT_23[r][c]); }

/* U[p, co, ci] = (G g G^T)[p].  Reference: cpu_winograd_weight_transform, src/backend/cpu/winograd/winograd_runtime.cpp:40-100 */
void oracle_winograd_weight_transform(int tile, int k, const float *w, float *u, int cout, int cin, int invert)
{
	const int p = tile + k - 1;
	for (int co = 0; co < cout; co++)
		for (int ci = 0; ci < cin; ci++)
		{
			double g[5][5], tmp[6][5];
			for (int r = 0; r < k; r++)
				for (int c = 0; c < k; c++)
				{
					const int rr = invert ? k - 1 - r : r, cc = invert ? k - 1 - c : c;
					g[r][c] = w[((size_t) (co * k + rr) * k + cc) * cin + ci];
				}
			for (int i = 0; i < p; i++)
				for (int c = 0; c < k; c++)
				{
					double s = 0.0;
					for (int r = 0; r < k; r++)
						s += g_at(tile, k, i, r) * g[r][c];
					tmp[i][c] = s;
				}
			for (int i = 0; i < p; i++)
				for (int j = 0; j < p; j++)
				{
					double s = 0.0;
					for (int c = 0; c < k; c++)
						s += tmp[i][c] * g_at(tile, k, j, c);
					u[((size_t) (i * p + j) * cout + co) * cin + ci] = (float) s;
				}
		}
}
/* V[p, tile, c] = (B^T d B)[p], zero padded patches.  Reference: winograd_runtime.cpp:101-160, tile order (b, th, tw) */
void oracle_winograd_input_transform(int tile, int k, const float *x, float *v, int batch, int height, int width, int channels)
{
	const int p = tile + k - 1, pad = k / 2;
	const int th_n = (height + tile - 1) / tile, tw_n = (width + tile - 1) / tile;
	const size_t tiles = (size_t) batch * th_n * tw_n;
	for (int b = 0; b < batch; b++)
		for (int th = 0; th < th_n; th++)
			for (int tw = 0; tw < tw_n; tw++)
			{
				const size_t t = ((size_t) b * th_n + th) * tw_n + tw;
				for (int c = 0; c < channels; c++)
				{
					double d[6][6], tmp[6][6];
					for (int r = 0; r < p; r++)
						for (int q = 0; q < p; q++)
						{
							const int h = tile * th - pad + r, w = tile * tw - pad + q;
							d[r][q] = (h >= 0 && h < height && w >= 0 && w < width) ? x[(((size_t) b * height + h) * width + w) * channels + c] : 0.0;
						}
					for (int i = 0; i < p; i++)
						for (int q = 0; q < p; q++)
						{
							double s = 0.0;
							for (int r = 0; r < p; r++)
								s += bt_at(p, i, r) * d[r][q];
							tmp[i][q] = s;
						}
					for (int i = 0; i < p; i++)
						for (int j = 0; j < p; j++)
						{
							double s = 0.0;
							for (int q = 0; q < p; q++)
								s += tmp[i][q] * bt_at(p, j, q);
							v[((size_t) (i * p + j) * tiles + t) * channels + c] = (float) s;
						}
				}
			}
}
/* y = act(A^T M A + ext + bias), clipped at the border.  Reference: winograd_runtime.cpp:161-230 */
void oracle_winograd_output_transform(int tile, int k, const float *m, float *y, const float *bias, const float *ext, int act, int batch,
		int height, int width, int channels)
{
	const int p = tile + k - 1;
	const int th_n = (height + tile - 1) / tile, tw_n = (width + tile - 1) / tile;
	const size_t tiles = (size_t) batch * th_n * tw_n;
	for (int b = 0; b < batch; b++)
		for (int th = 0; th < th_n; th++)
			for (int tw = 0; tw < tw_n; tw++)
			{
				const size_t t = ((size_t) b * th_n + th) * tw_n + tw;
				for (int c = 0; c < channels; c++)
				{
					double tmp[4][6];
					for (int i = 0; i < tile; i++)
						for (int q = 0; q < p; q++)
						{
							double s = 0.0;
							for (int r = 0; r < p; r++)
								s += at_at(tile, k, i, r) * m[((size_t) (r * p + q) * tiles + t) * channels + c];
							tmp[i][q] = s;
						}
					for (int i = 0; i < tile; i++)
						for (int j = 0; j < tile; j++)
						{
							const int h = tile * th + i, w = tile * tw + j;
							if (h >= height || w >= width)
								continue;
							double s = 0.0;
							for (int q = 0; q < p; q++)
								s += tmp[i][q] * at_at(tile, k, j, q);
							const size_t off = (((size_t) b * height + h) * width + w) * channels + c;
							float r = (float) s;
							if (ext != NULL)
								r += ext[off];
							if (bias != NULL)
								r += bias[c];
							y[off] = activate(r, act);
						}
				}
			}
}

/* ---------------------------------------------------------------------------------------------------------------
 * GEMM, row-major: C (rows x cols) = alpha * op(A) * op(B) + beta * C.  Reference semantics: cpu_gemm,
 * src/backend/cpu/gemm/gemm.cpp and the naive baselines of test/backend/test_gemms.cpp:31-90.
 * ------------------------------------------------------------------------------------------------------------- */
void oracle_gemm(int trans_a, int trans_b, int rows, int cols, int k, float alpha, const float *a, int lda, const float *b, int ldb,
		float beta, float *c, int ldc)
{
#pragma omp parallel for
	for (int i = 0; i < rows; i++)
		for (int j = 0; j < cols; j++)
		{
			double s = 0.0;
			for (int l = 0; l < k; l++)
			{
				const float av = trans_a ? a[(size_t) l * lda + i] : a[(size_t) i * lda + l];
				const float bv = trans_b ? b[(size_t) j * ldb + l] : b[(size_t) l * ldb + j];
				s += (double) av * bv;
			}
			float r = alpha * (float) s;
			if (beta != 0.0f)
				r += beta * c[(size_t) i * ldc + j];
			c[(size_t) i * ldc + j] = r;
		}
}
/* int8 x int8 -> int32, exact.  Reference: the int8 'n','t' product of src/layers/Conv2D.cpp:232 */
void oracle_gemm_i8_nt(int rows, int cols, int k, const int8_t *a, const int8_t *b, int32_t *c)
{
#pragma omp parallel for
	for (int i = 0; i < rows; i++)
		for (int j = 0; j < cols; j++)
		{
			int32_t s = 0;
			for (int l = 0; l < k; l++)
				s += (int32_t) a[(size_t) i * k + l] * (int32_t) b[(size_t) j * k + l];
			c[(size_t) i * cols + j] = s;
		}
}

/* ---------------------------------------------------------------------------------------------------------------
 * Direct convolution, stride 1, "same" zero padding: y = act(conv(x, w) + bias + ext).
 * Reference: baseline_conv2D_forward, test/backend/test_conv2D.cpp:22-59.
 * ------------------------------------------------------------------------------------------------------------- */
void oracle_conv2d(const float *x, const float *w, const float *bias, const float *ext, float *y, int act, int batch, int height, int width,
		int cin, int cout, int k)
{
	const int pad = (k - 1) / 2;
#pragma omp parallel for collapse(2)
	for (int b = 0; b < batch; b++)
		for (int h = 0; h < height; h++)
			for (int wd = 0; wd < width; wd++)
				for (int co = 0; co < cout; co++)
				{
					double s = 0.0;
					for (int i = 0; i < k; i++)
						for (int j = 0; j < k; j++)
						{
							const int ih = h - pad + i, iw = wd - pad + j;
							if (ih < 0 || ih >= height || iw < 0 || iw >= width)
								continue;
							const float *px = x + (((size_t) b * height + ih) * width + iw) * cin;
							const float *pw = w + ((size_t) (co * k + i) * k + j) * cin;
							for (int ci = 0; ci < cin; ci++)
								s += (double) px[ci] * pw[ci];
						}
					const size_t off = (((size_t) b * height + h) * width + wd) * cout + co;
					float r = (float) s;
					if (bias != NULL)
						r += bias[co];
					if (ext != NULL)
						r += ext[off];
					y[off] = activate(r, act);
				}
}

/* ---------------------------------------------------------------------------------------------------------------
 * int8 convolution.  Restates the scalar loop of src/layers/Conv2D.cpp:240-308: taps outside the image contribute
 * weight * input_zero; x = acc * channel_scale[co] + bias[co] (+ ext * ext_scale + ext_shift); activation;
 * int8 output = clamp(round(x * (1 / out_scale) + (-out_shift / out_scale))).  `acc_out` (may be NULL) receives
 * the raw int32 accumulators -- the values the CUDA path must reproduce bit for bit.
 * ------------------------------------------------------------------------------------------------------------- */
static int32_t quantize_i8(float x)
{ /* reference: quantize(), src/layers/quantization.cpp:43-47 */
	float r = roundf(x);
	if (r < -128.0f) r = -128.0f;
	if (r > 127.0f) r = 127.0f;
	return (int32_t) r;
}
void oracle_conv2d_int8(const int8_t *x, const int8_t *w, const float *channel_scales, const float *bias, const int8_t *ext, float ext_scale,
		float ext_shift, int32_t input_zero, float out_scale, float out_shift, int act, int8_t *y_i8, float *y_f32, int32_t *acc_out, int batch,
		int height, int width, int cin, int cout, int k)
{
	const int pad = (k - 1) / 2;
	const float inv_scale = 1.0f / out_scale, inv_shift = -out_shift / out_scale; /* AffineTransform::get_inverse */
#pragma omp parallel for collapse(2)
	for (int b = 0; b < batch; b++)
		for (int h = 0; h < height; h++)
			for (int wd = 0; wd < width; wd++)
				for (int co = 0; co < cout; co++)
				{
					int32_t acc = 0;
					for (int i = 0; i < k; i++)
						for (int j = 0; j < k; j++)
						{
							const int ih = h - pad + i, iw = wd - pad + j;
							const int8_t *pw = w + ((size_t) (co * k + i) * k + j) * cin;
							if (ih >= 0 && ih < height && iw >= 0 && iw < width)
							{
								const int8_t *px = x + (((size_t) b * height + ih) * width + iw) * cin;
								for (int ci = 0; ci < cin; ci++)
									acc += (int32_t) pw[ci] * (int32_t) px[ci];
							}
							else
								for (int ci = 0; ci < cin; ci++)
									acc += (int32_t) pw[ci] * input_zero;
						}
					const size_t off = (((size_t) b * height + h) * width + wd) * cout + co;
					if (acc_out != NULL)
						acc_out[off] = acc;
					float tmp = (float) acc * channel_scales[co] + bias[co];
					if (ext != NULL)
						tmp += (float) ext[off] * ext_scale + ext_shift;
					if (act == ACT_SIGMOID || act == ACT_TANH || act == ACT_RELU || act == ACT_EXP)
						tmp = activate(tmp, act);
					if (y_i8 != NULL)
						y_i8[off] = (int8_t) quantize_i8(tmp * inv_scale + inv_shift);
					if (y_f32 != NULL)
						y_f32[off] = tmp;
				}
}
/* Per-output-channel symmetric weight quantisation.  Restates quantize_weights, src/layers/quantization.cpp:59-97:
 * s = 127 / max|w_co|;  q = clamp(round(w * s));  channel_scale = in_scale / s;  bias' = in_shift / s * sum(q) + bias. */
void oracle_quantize_weights(const float *w, const float *bias, float in_scale, float in_shift, int8_t *q, float *channel_scales,
		float *q_bias, int cout, int per_filter)
{
	for (int co = 0; co < cout; co++)
	{
		float max_abs = 0.0f;
		for (int j = 0; j < per_filter; j++)
		{
			const float a = fabsf(w[(size_t) co * per_filter + j]);
			if (a > max_abs) max_abs = a;
		}
		const float s = 127.0f / max_abs;
		channel_scales[co] = in_scale / s;
		int32_t sum_q = 0;
		for (int j = 0; j < per_filter; j++)
		{
			const int32_t v = quantize_i8(w[(size_t) co * per_filter + j] * s);
			sum_q += v;
			q[(size_t) co * per_filter + j] = (int8_t) v;
		}
		q_bias[co] = in_shift / s * (float) sum_q + (bias != NULL ? bias[co] : 0.0f);
	}
}
/* int32 accumulators -> fp32 or int8.  Restates kernel_scale_shift_act, src/backend/cuda/kernels/quantized.cu:219-257
 * (the only implementation: the CPU dispatcher has none, src/core/math.cpp:1556-1574). */
void oracle_scale_shift_act(const int32_t *acc, const float *scales, const float *bias, const int8_t *ext, float ext_scale, float ext_shift,
		float out_scale, float out_shift, int act, int8_t *y_i8, float *y_f32, size_t rows, int channels)
{
	for (size_t i = 0; i < rows; i++)
		for (int c = 0; c < channels; c++)
		{
			const size_t off = i * channels + c;
			float x = (float) acc[off] * scales[c] + bias[c];
			if (ext != NULL)
				x += (float) ext[off] * ext_scale + ext_shift;
			if (act == ACT_SIGMOID || act == ACT_TANH || act == ACT_RELU)
				x = activate(x, act);
			if (y_f32 != NULL)
				y_f32[off] = x;
			if (y_i8 != NULL)
				y_i8[off] = (int8_t) quantize_i8((x - out_shift) / out_scale);
		}
}
/* [b,h,w,c] -> [b*h*w, k*k*c] with columns (kh, kw, c); elem = bytes per element; pad = one element.
 * Reference: baseline_receptive_fields, test/backend/test_gemm_conv.cpp:17-62. */
void oracle_im2row(const uint8_t *x, uint8_t *out, int batch, int height, int width, int channels, int k, int invert, int elem,
		const uint8_t *pad)
{
	const int p = (k - 1) / 2;
	size_t o = 0;
	for (int b = 0; b < batch; b++)
		for (int h = 0; h < height; h++)
			for (int w = 0; w < width; w++)
				for (int i = 0; i < k; i++)
					for (int j = 0; j < k; j++)
					{
						const int ih = h - p + (invert ? k - 1 - i : i), iw = w - p + (invert ? k - 1 - j : j);
						for (int c = 0; c < channels; c++, o += elem)
						{
							if (ih >= 0 && ih < height && iw >= 0 && iw < width)
								memcpy(out + o, x + ((((size_t) b * height + ih) * width + iw) * channels + c) * elem, elem);
							else if (pad != NULL)
								memcpy(out + o, pad, elem);
							else
								memset(out + o, 0, elem);
						}
					}
}

/* ---------------------------------------------------------------------------------------------------------------
 * Pooling, normalisation, attention, input unpacking.
 * ------------------------------------------------------------------------------------------------------------- */
/* Reference: cpu_global_average_pooling_forward, src/backend/cpu/kernels/pooling_and_scaling.cpp */
void oracle_global_average_pooling(const float *x, float *y, float alpha, float beta, int batch, int hw, int channels)
{
	for (int b = 0; b < batch; b++)
		for (int c = 0; c < channels; c++)
		{
			double s = 0.0;
			for (int i = 0; i < hw; i++)
				s += x[((size_t) b * hw + i) * channels + c];
			float r = alpha * (float) (s / hw);
			if (beta != 0.0f)
				r += beta * y[(size_t) b * channels + c];
			y[(size_t) b * channels + c] = r;
		}
}
/* Reference: cpu_layernorm_forward, src/backend/cpu/normalization.cpp:346-397 (ext added first; unbiased variance; eps 1e-6) */
void oracle_layernorm(const float *x, float *y, const float *gamma, const float *beta, const float *ext, size_t rows, int channels)
{
	for (size_t r = 0; r < rows; r++)
	{
		double mean = 0.0, var = 0.0;
		for (int j = 0; j < channels; j++)
			mean += x[r * channels + j] + (ext != NULL ? ext[r * channels + j] : 0.0f);
		mean /= channels;
		for (int j = 0; j < channels; j++)
		{
			const double d = x[r * channels + j] + (ext != NULL ? ext[r * channels + j] : 0.0f) - mean;
			var += d * d;
		}
		const double stddev = sqrt(1.0e-6 + var / (channels - 1));
		for (int j = 0; j < channels; j++)
		{
			const double v = x[r * channels + j] + (ext != NULL ? ext[r * channels + j] : 0.0f);
			y[r * channels + j] = (float) ((gamma != NULL ? gamma[j] : 1.0f) * (v - mean) / stddev + (beta != NULL ? beta[j] : 0.0f));
		}
	}
}
/* Reference: cpu_multi_head_attention_forward + softmax_forward_in_place, src/backend/cpu/attention.cpp:143-208,394-434;
 * baseline_mha_forward, test/backend/test_attention.cpp:273-300.  x [b, T, parts, heads, d]; table [heads, n, round_up(n,4)] */
void oracle_mha_forward(const float *x, float *y, const float *table, int batch, int height, int width, int heads, int head_dim,
		int symmetric, int table_n)
{
	const int tokens = height * width, parts = symmetric ? 2 : 3;
	const int stride = parts * heads * head_dim, pad_n = (table_n + 3) / 4 * 4, range = (table_n - 1) / 2;
	const double scale = 1.0 / sqrt((double) head_dim);
#pragma omp parallel for collapse(2)
	for (int b = 0; b < batch; b++)
		for (int h = 0; h < heads; h++)
		{
			double *s = (double*) malloc(sizeof(double) * tokens);
			const float *base = x + (size_t) b * tokens * stride;
			for (int i = 0; i < tokens; i++)
			{
				const float *q = base + (size_t) i * stride + h * head_dim;
				double mx = -1.0e300;
				for (int j = 0; j < tokens; j++)
				{
					const float *kk = base + (size_t) j * stride + (symmetric ? 0 : 1) * heads * head_dim + h * head_dim;
					double acc = 0.0;
					for (int d = 0; d < head_dim; d++)
						acc += (double) q[d] * kk[d];
					acc *= scale;
					if (table != NULL)
					{
						int dh = j / width - i / width, dw = j % width - i % width;
						dh = dh < -range ? -range : (dh > range ? range : dh);
						dw = dw < -range ? -range : (dw > range ? range : dw);
						acc += table[((size_t) h * table_n + (range + dh)) * pad_n + (range + dw)];
					}
					s[j] = acc;
					if (acc > mx) mx = acc;
				}
				double sum = 0.0;
				for (int j = 0; j < tokens; j++)
				{
					s[j] = exp(s[j] - mx);
					sum += s[j];
				}
				for (int d = 0; d < head_dim; d++)
				{
					double o = 0.0;
					for (int j = 0; j < tokens; j++)
						o += s[j] * base[(size_t) j * stride + (parts - 1) * heads * head_dim + h * head_dim + d];
					y[((size_t) b * tokens + i) * heads * head_dim + h * head_dim + d] = (float) (o / sum);
				}
			}
			free(s);
		}
}
/* Reference: cpu_unpack_input, src/backend/cpu/def_misc_kernels.cpp; channel j of a position = bit (j % 32) of word j / 32 */
void oracle_unpack_input(const uint32_t *packed, float *y, size_t rows, int channels)
{
	const int words = (channels + 31) / 32;
	for (size_t r = 0; r < rows; r++)
		for (int j = 0; j < channels; j++)
			y[r * channels + j] = ((packed[r * words + j / 32] >> (j % 32)) & 1u) ? 1.0f : 0.0f;
}
void oracle_softmax(const float *x, float *y, size_t rows, int channels)
{
	for (size_t r = 0; r < rows; r++)
	{
		double mx = -1.0e300, sum = 0.0;
		for (int j = 0; j < channels; j++)
			if (x[r * channels + j] > mx) mx = x[r * channels + j];
		for (int j = 0; j < channels; j++)
			sum += exp(x[r * channels + j] - mx);
		for (int j = 0; j < channels; j++)
			y[r * channels + j] = (float) (exp(x[r * channels + j] - mx) / sum);
	}
}
/* y = act(x + bias[c]) -- reference: cpu_add_bias_act, src/backend/cpu/dispatcher.cpp */
void oracle_add_bias_act(const float *x, const float *bias, float *y, int act, size_t rows, int channels)
{
	for (size_t r = 0; r < rows; r++)
		for (int c = 0; c < channels; c++)
			y[r * channels + c] = activate(x[r * channels + c] + (bias != NULL ? bias[c] : 0.0f), act);
}

/* ---------------------------------------------------------------------------------------------------------------
 * Layers adjacent to the convolution path (batch norm at inference time, depthwise convolution, channel scaling).
 * ------------------------------------------------------------------------------------------------------------- */

/* y = alpha * act(x * scale[c] + shift[c]) + beta * y with scale = gamma / sqrt(var + 1e-6), shift = beta_bn - mean * scale;
 * avg_var = [mean[channels], var[channels]]  (src/backend/cuda/kernels/batchnorm.cu:58-100; CPU: src/backend/cpu/normalization.cpp) */
void oracle_batchnorm_inference(const float *x, float *y, const float *gamma, const float *beta_bn, const float *avg_var, float alpha,
		float beta, int act, size_t rows, int channels)
{
	for (size_t r = 0; r < rows; r++)
		for (int c = 0; c < channels; c++)
		{
			const float scale = (gamma ? gamma[c] : 1.0f) / sqrtf(avg_var[channels + c] + 1.0e-6f);
			const float shift = -avg_var[c] * scale + (beta_bn ? beta_bn[c] : 0.0f);
			float v = activate(x[r * channels + c] * scale + shift, act) * alpha;
			if (beta != 0.0f)
				v += beta * y[r * channels + c];
			y[r * channels + c] = v;
		}
}
/* Folds the same scale / shift into a layer: weights [outer, inner]; per_row != 0: one channel per row ([cout, ...] weights),
 * else one channel per column (depthwise [k*k, c])  (batchnorm.cu:400-438, src/backend/cpu/normalization.cpp cpu_fold_batchnorm) */
void oracle_fold_batchnorm(float *weights, float *bias, const float *gamma, const float *beta_bn, const float *avg_var, int outer, int inner,
		int per_row)
{
	const int channels = per_row ? outer : inner;
	for (int c = 0; c < channels; c++)
	{
		const float scale = (gamma ? gamma[c] : 1.0f) / sqrtf(avg_var[channels + c] + 1.0e-6f);
		const float shift = -avg_var[c] * scale + (beta_bn ? beta_bn[c] : 0.0f);
		if (per_row)
			for (int i = 0; i < inner; i++)
				weights[(size_t) c * inner + i] *= scale;
		else
			for (int i = 0; i < outer; i++)
				weights[(size_t) i * inner + c] *= scale;
		if (bias)
			bias[c] = bias[c] * scale + shift;
	}
}
/* y = alpha * dwconv(x, w) + bias + beta * y; x [b,h,w,c], w [k,k,c], stride 1, zero "same" padding (depthwise_conv.cu:110-182) */
void oracle_depthwise_conv(const float *x, const float *w, const float *bias, float *y, float alpha, float beta, int batch, int height,
		int width, int channels, int k)
{
	const int pad = (k - 1) / 2;
	for (int b = 0; b < batch; b++)
		for (int h = 0; h < height; h++)
			for (int q = 0; q < width; q++)
				for (int c = 0; c < channels; c++)
				{
					double acc = 0.0;
					for (int i = 0; i < k; i++)
						for (int j = 0; j < k; j++)
						{
							const int hh = h + i - pad, ww = q + j - pad;
							if (hh >= 0 && hh < height && ww >= 0 && ww < width)
								acc += (double) x[(((size_t) b * height + hh) * width + ww) * channels + c] * (double) w[((size_t) i * k + j) * channels + c];
						}
					const size_t off = (((size_t) b * height + h) * width + q) * channels + c;
					float v = (float) acc * alpha + (bias ? bias[c] : 0.0f);
					if (beta != 0.0f)
						v += beta * y[off];
					y[off] = v;
				}
}
/* The integer branch of DepthwiseConv2D::forward on the CPU (src/layers/DepthwiseConv2D.cpp:104-140): the accumulator starts at 0,
 * positions outside the image contribute weight * input_zero, then acc * scale[c] + bias[c], requantised with the inverse transform. */
void oracle_depthwise_conv_int8(const int8_t *x, const int8_t *w, const float *scales, const float *bias, int8_t *y_i8, float *y_f32,
		float out_scale, float out_shift, int input_zero, int batch, int height, int width, int channels, int k)
{
	const int pad = (k - 1) / 2;
	const float inv_scale = 1.0f / out_scale, inv_shift = -out_shift / out_scale;
	for (int b = 0; b < batch; b++)
		for (int h = 0; h < height; h++)
			for (int q = 0; q < width; q++)
				for (int c = 0; c < channels; c++)
				{
					int32_t acc = 0;
					for (int i = 0; i < k; i++)
						for (int j = 0; j < k; j++)
						{
							const int hh = h + i - pad, ww = q + j - pad;
							const int wv = w[((size_t) i * k + j) * channels + c];
							if (hh >= 0 && hh < height && ww >= 0 && ww < width)
								acc += wv * (int) x[(((size_t) b * height + hh) * width + ww) * channels + c];
							else
								acc += wv * input_zero;
						}
					const size_t off = (((size_t) b * height + h) * width + q) * channels + c;
					const float tmp = (float) acc * (scales ? scales[c] : 1.0f) + (bias ? bias[c] : 0.0f);
					if (y_f32)
						y_f32[off] = tmp;
					if (y_i8)
						y_i8[off] = (int8_t) quantize_i8(tmp * inv_scale + inv_shift);
				}
}
/* y = alpha * x * s[b, c] + beta * y; x [b, hw, c], s [b, c]  (src/backend/cuda/kernels/global_pooling.cu:99-123) */
void oracle_channel_scaling(const float *x, const float *scales, float *y, float alpha, float beta, int batch, int hw, int channels)
{
	for (int b = 0; b < batch; b++)
		for (int i = 0; i < hw; i++)
			for (int c = 0; c < channels; c++)
			{
				const size_t off = ((size_t) b * hw + i) * channels + c;
				float v = x[off] * scales[(size_t) b * channels + c] * alpha;
				if (beta != 0.0f)
					v += beta * y[off];
				y[off] = v;
			}
}

/* ---------------------------------------------------------------------------------------------------------------
 * Backward pass of the Winograd convolution: gradient transform (dy tiles -> matrices), update transform
 * (accumulated matrices -> weight gradient) and the fused activation-backward / bias-gradient / copy step.
 * Matrices restated from src/backend/cuda/kernels/winograd_transforms.cuh:95-135 (F(2x2,3x3)), :205-250 (F(4x4,3x3)),
 * :304-352 (F(2x2,5x5)); the CPU twins are src/backend/cpu/winograd/def_winograd_kernels.cpp.
 * ------------------------------------------------------------------------------------------------------------- */
static const double GR_23[4][2] = { { 1, 0 }, { 1, 1 }, { 1, -1 }, { 0, 1 } };
static const double GR_43[6][4] = { { 1, 0, 0, 0 }, { 2.0 / 3, 2.0 / 3, 2.0 / 3, 2.0 / 3 }, { 2.0 / 3, -2.0 / 3, 2.0 / 3, -2.0 / 3 },
		{ 1.0 / 3, 2.0 / 3, 4.0 / 3, 8.0 / 3 }, { 1.0 / 3, -2.0 / 3, 4.0 / 3, -8.0 / 3 }, { 0, 0, 0, 2 } };
static const double GR_25[6][2] = { { 1, 0 }, { 2.0 / 3, 2.0 / 3 }, { 2.0 / 3, -2.0 / 3 }, { 1.0 / 3, 2.0 / 3 }, { 1.0 / 3, -2.0 / 3 }, { 0, 1 } };
static const double UP_23[3][4] = { { 1, 0.5, 0.5, 0 }, { 0, 0.5, -0.5, 0 }, { 0, 0.5, 0.5, 1 } };
static const double UP_43[3][6] = { { 1, 1, 1, 0.25, 0.25, 0 }, { 0, 1, -1, 0.5, -0.5, 0 }, { 0, 1, 1, 1, 1, 2 } };
static const double UP_25[5][6] = { { 1, 1, 1, 0.25, 0.25, 0 }, { 0, 1, -1, 0.5, -0.5, 0 }, { 0, 1, 1, 1, 1, 0 }, { 0, 1, -1, 2, -2, 0 },
		{ 0, 1, 1, 4, 4, 4 } };
static double gr_at(int tile, int k, int r, int c) { return k == 5 ? GR_25[r][c] : (tile == 4 ? GR_43[r][c] : GR_23[r][c]); }
static double up_at(int tile, int k, int r, int c) { return k == 5 ? UP_25[r][c] : (tile == 4 ? UP_43[r][c] : UP_23[r][c]); }

/* M[p, tile, c] = (Gr d Gr^T)[p] for the tile x tile pieces of dy (zero beyond the border), tile order (b, th, tw)
 * (winograd_nonfused.cu:182-212) */
void oracle_winograd_gradient_transform(int tile, int k, const float *dy, float *m, int batch, int height, int width, int channels)
{
	const int p = tile + k - 1;
	const int th_n = (height + tile - 1) / tile, tw_n = (width + tile - 1) / tile;
	const size_t tiles = (size_t) batch * th_n * tw_n;
	for (int b = 0; b < batch; b++)
		for (int th = 0; th < th_n; th++)
			for (int tw = 0; tw < tw_n; tw++)
			{
				const size_t t = ((size_t) b * th_n + th) * tw_n + tw;
				for (int c = 0; c < channels; c++)
				{
					double d[4][4], tmp[6][4];
					for (int r = 0; r < tile; r++)
						for (int q = 0; q < tile; q++)
						{
							const int h = tile * th + r, w = tile * tw + q;
							d[r][q] = (h < height && w < width) ? dy[(((size_t) b * height + h) * width + w) * channels + c] : 0.0;
						}
					for (int i = 0; i < p; i++)
						for (int q = 0; q < tile; q++)
						{
							double s = 0.0;
							for (int r = 0; r < tile; r++)
								s += gr_at(tile, k, i, r) * d[r][q];
							tmp[i][q] = s;
						}
					for (int i = 0; i < p; i++)
						for (int j = 0; j < p; j++)
						{
							double s = 0.0;
							for (int q = 0; q < tile; q++)
								s += tmp[i][q] * gr_at(tile, k, j, q);
							m[((size_t) (i * p + j) * tiles + t) * channels + c] = (float) s;
						}
				}
			}
}
/* dw[co, :, :, ci] = Up M[:, co, ci] Up^T with M [p*p, cout, cin] (winograd_nonfused.cu:214-239) */
void oracle_winograd_update_transform(int tile, int k, const float *m, float *dw, int cout, int cin)
{
	const int p = tile + k - 1;
	for (int co = 0; co < cout; co++)
		for (int ci = 0; ci < cin; ci++)
		{
			double d[6][6], tmp[5][6];
			for (int r = 0; r < p; r++)
				for (int q = 0; q < p; q++)
					d[r][q] = m[((size_t) (r * p + q) * cout + co) * cin + ci];
			for (int i = 0; i < k; i++)
				for (int q = 0; q < p; q++)
				{
					double s = 0.0;
					for (int r = 0; r < p; r++)
						s += up_at(tile, k, i, r) * d[r][q];
					tmp[i][q] = s;
				}
			for (int i = 0; i < k; i++)
				for (int j = 0; j < k; j++)
				{
					double s = 0.0;
					for (int q = 0; q < p; q++)
						s += tmp[i][q] * up_at(tile, k, j, q);
					dw[(((size_t) co * k + i) * k + j) * cin + ci] = (float) s;
				}
		}
}
/* dy <- dy * act'(y) (in place); db <- beta_db * db + column sums of the new dy; dx <- dy + beta_dx * dx
 * (src/backend/cuda/kernels/tensor_op.cu:195-270,527-580; the CPU backend has no counterpart) */
void oracle_act_bias_copy_backward(float *dy, const float *y, float *dx, float *db, float beta_dx, float beta_db, int act, size_t rows,
		int channels)
{
	if (db)
		for (int c = 0; c < channels; c++)
			db[c] *= beta_db;
	for (int c = 0; c < channels; c++)
	{
		double sum = 0.0;
		for (size_t r = 0; r < rows; r++)
		{
			const size_t i = r * channels + c;
			float g = dy[i];
			switch (act)
			{
				case 1:
					g *= y[i] * (1.0f - y[i]);
					break;
				case 2:
					g *= 1.0f - y[i] * y[i];
					break;
				case 3:
					g = (y[i] > 0.0f) ? g : 0.0f;
					break;
				case 4:
					g = (y[i] > 0.0f) ? g : g * 0.1f;
					break;
				default:
					break;
			}
			dy[i] = g;
			sum += g;
			if (dx)
				dx[i] = (beta_dx != 0.0f) ? g + beta_dx * dx[i] : g;
		}
		if (db)
			db[c] += (float) sum;
	}
}

/* ---------------------------------------------------------------------------------------------------------------
 * Layers between the convolution blocks: RMS normalisation and the space <-> depth rearrangements.
 * --------------------------------------------------------------------------------------------------------------- */
/* y[r, c] = gamma[c] * x[r, c] / (1e-6 + sqrt(mean_c x^2))  (src/backend/cpu/normalization.cpp:452-486; gamma may be NULL) */
void oracle_rmsnorm(const float *x, float *y, const float *gamma, size_t rows, int channels)
{
	for (size_t r = 0; r < rows; r++)
	{
		float sum = 0.0f;
		for (int c = 0; c < channels; c++)
			sum += x[r * channels + c] * x[r * channels + c];
		const float inv_rms = 1.0f / (1.0e-6f + sqrtf(sum / (float) channels));
		for (int c = 0; c < channels; c++)
			y[r * channels + c] = (gamma ? gamma[c] : 1.0f) * x[r * channels + c] * inv_rms;
	}
}
/* The smallest p with ceil(larger / p) == smaller, 0 if none (src/backend/cpu/dispatcher.cpp:125-137). */
static int patch_size(int smaller, int larger)
{
	for (int p = 1; smaller > 0 && larger >= smaller; p++)
	{
		const int tmp = (larger + p - 1) / p;
		if (tmp == smaller)
			return p;
		if (tmp < smaller)
			break;
	}
	return 0;
}
/* [b, h, w, c] -> [b, oh, ow, p*q*c] with zero fill past the edge; element size in bytes so that any dtype can be checked
 * (src/backend/cpu/dispatcher.cpp:190-219). Returns 0 when the shapes do not fit. */
int oracle_space_to_depth(const uint8_t *x, uint8_t *y, int elem, int batch, int h, int w, int c, int oh, int ow)
{
	const int p = patch_size(oh, h), q = patch_size(ow, w);
	if (p == 0 || q == 0)
		return 0;
	const size_t block = (size_t) elem * c;
	for (int b = 0; b < batch; b++)
		for (int i = 0; i < oh; i++)
			for (int j = 0; j < ow; j++)
				for (int dx = 0; dx < p; dx++)
					for (int dy = 0; dy < q; dy++)
					{
						const int hh = i * p + dx, ww = j * q + dy;
						if (hh < h && ww < w)
							memcpy(y, x + (((size_t) b * h + hh) * w + ww) * block, block);
						else
							memset(y, 0, block);
						y += block;
					}
	return 1;
}
/* The inverse: [b, ih, iw, p*q*c] -> [b, h, w, c]  (src/backend/cpu/dispatcher.cpp:220-247). */
int oracle_depth_to_space(const uint8_t *x, uint8_t *y, int elem, int batch, int ih, int iw, int h, int w, int c)
{
	const int p = patch_size(ih, h), q = patch_size(iw, w);
	if (p == 0 || q == 0)
		return 0;
	const size_t block = (size_t) elem * c;
	for (int b = 0; b < batch; b++)
		for (int i = 0; i < ih; i++)
			for (int j = 0; j < iw; j++)
				for (int dx = 0; dx < p; dx++)
					for (int dy = 0; dy < q; dy++)
					{
						const int hh = i * p + dx, ww = j * q + dy;
						if (hh < h && ww < w)
							memcpy(y + (((size_t) b * h + hh) * w + ww) * block, x, block);
						x += block;
					}
	return 1;
}
