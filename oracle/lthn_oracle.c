/*
 * lthn_oracle.c — CPU restatement of go-inference's MLX-affine quantized-linear
 * path and the small transformer references around it.
 *
 * THIS FILE IS TEST INFRASTRUCTURE. It is the checker the CUDA kernels are
 * compared against and the timed CPU baseline; nothing in the shipped library
 * links, loads or calls it.
 *
 * Parity status: PINNED to the reference's own known-answer tests (see
 * tests/test_oracle_kat.py): enginetest/quant_reference_test.go:13-38 (12.5),
 * engine/hip/hip_projection_reference_test.go:71-110 ([28,38], [120,136],
 * [10,26]), enginetest/quant_parity.go:33-67 (formula fixture),
 * model/quant/mlxaffine/mlxaffine_test.go (round-trip bound, code fixed point,
 * constant group, shape contract, rejected widths) and cross-checked against
 * golden vectors produced by the reference's own tools/mlxaffine_dequant.py.
 * The reference's Go sources cannot be compiled where this was written (no Go
 * toolchain), so every function below follows the cited Go text line by line.
 * UNPINNED: byte identity with mlx_lm.convert output (the reference pins that
 * only against a Hugging Face snapshot that is not available offline,
 * model/quant/mlxaffine/oracle_test.go:49-106).
 *
 * All paths are relative to the reference's `go/` directory.
 * Build: see oracle/Makefile (gcc -O2 -ffp-contract=off -fopenmp).
 * -ffp-contract=off matters: Go on amd64 never fuses a*b+c, so neither may we.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define LTHN_O_OK 0
#define LTHN_O_EINVAL 1

/* ------------------------------------------------------------------ bf16 -- */

static inline float f32_from_bits(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }
static inline uint32_t f32_bits(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }

/* model/quant/mlxaffine/mlxaffine.go:229-236 float32ToBFloat16 (RNE, quiet NaN);
 * identical to enginetest/quant_reference.go:28-35 bf16Encode. */
uint16_t lthn_o_f32_to_bf16(float f) {
    uint32_t u = f32_bits(f);
    if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x0040u);
    u += 0x7fffu + ((u >> 16) & 1u);
    return (uint16_t)(u >> 16);
}

/* mlxaffine.go:241 bfloat16ToFloat32 / quant_reference.go:23-25 bf16Decode. */
float lthn_o_bf16_to_f32(uint16_t h) { return f32_from_bits((uint32_t)h << 16); }

void lthn_o_round_bf16_inplace(float *v, long n) {
    /* engine/hip/hip_gemma4_q4_oracle_test.go:850-858 hipOracleRoundBF16 */
    for (long i = 0; i < n; i++) {
        uint32_t b = f32_bits(v[i]);
        b += 0x7fffu + ((b >> 16) & 1u);
        v[i] = f32_from_bits(b & 0xffff0000u);
    }
}

int lthn_o_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

/* ------------------------------------------------- a1: QuantizeTensor ---- */

/* mlxaffine.go:213 roundHalfAway: math.Round(float64(v)) — ties away from 0. */
static inline float round_half_away(float v) { return (float)round((double)v); }
static inline float abs32(float x) { return x < 0 ? -x : x; } /* mlxaffine.go:217-222 */

static int supported_bits(int bits) { /* mlxaffine.go:56 SupportedBits */
    return bits == 1 || bits == 2 || bits == 4 || bits == 8;
}

/* mlxaffine.go:136-161 affineGroup (edge-anchored MLX rule), variant 0.
 * variant 1 is the literal rule a benchmark configuration states in prose:
 * scale=(max-min)/nBins (floored at 1e-7), bias=min. */
static void affine_group(const float *g, int n, float nbins, int variant, float *scale_out, float *bias_out) {
    float wmin = g[0], wmax = g[0];
    for (int i = 1; i < n; i++) {
        float v = g[i];
        if (v < wmin) wmin = v;
        if (v > wmax) wmax = v;
    }
    float scale = (wmax - wmin) / nbins;
    const float eps = 1e-7f; /* mlxaffine.go:49 affineEps */
    if (scale < eps) scale = eps;
    if (variant == 1) { *scale_out = scale; *bias_out = wmin; return; }
    float edge = wmax;
    if (abs32(wmin) > abs32(wmax)) edge = wmin; else scale = -scale;
    float q0 = round_half_away(edge / scale);
    if (q0 == 0) { *scale_out = scale; *bias_out = 0; return; }
    *scale_out = edge / q0;
    *bias_out = edge;
}

/* mlxaffine.go:165-173 quantiseCode */
static inline uint32_t quantise_code(float x, float bias, float scale, float nbins) {
    float q = round_half_away((x - bias) / scale);
    if (q < 0) q = 0; else if (q > nbins) q = nbins;
    return (uint32_t)q;
}

/* mlxaffine.go:80-129 QuantizeTensor. packed: outDim*inDim*bits/8 bytes (LE u32
 * words), scales/biases: outDim*(inDim/gs) bf16. Rows are independent, so the
 * row loop is OpenMP-parallel; per-row arithmetic is the reference's. */
int lthn_o_quantize(const float *values, long out_dim, long in_dim, int bits, int gs, int variant,
                    uint8_t *packed, uint16_t *scales, uint16_t *biases) {
    if (!supported_bits(bits)) return LTHN_O_EINVAL;
    if (out_dim <= 0 || in_dim <= 0) return LTHN_O_EINVAL;
    if (gs <= 0 || in_dim % gs != 0) return LTHN_O_EINVAL;
    int epw = 32 / bits;
    if (gs % epw != 0) return LTHN_O_EINVAL;
    long wpr = in_dim * bits / 32, wpg = gs / epw, gpr = in_dim / gs;
    float nbins = (float)((1 << bits) - 1);
    uint32_t *words = (uint32_t *)packed;
#pragma omp parallel for schedule(static)
    for (long r = 0; r < out_dim; r++) {
        for (long g = 0; g < gpr; g++) {
            const float *grp = values + r * in_dim + g * gs;
            float scale, bias;
            affine_group(grp, gs, nbins, variant, &scale, &bias);
            scales[r * gpr + g] = lthn_o_f32_to_bf16(scale);
            biases[r * gpr + g] = lthn_o_f32_to_bf16(bias);
            for (long wg = 0; wg < wpg; wg++) {
                uint32_t word = 0;
                for (int p = 0; p < epw; p++)
                    word |= quantise_code(grp[wg * epw + p], bias, scale, nbins) << (p * bits);
                words[r * wpr + g * wpg + wg] = word; /* little-endian host */
            }
        }
    }
    return LTHN_O_OK;
}

/* ------------------------------------------------ a2: DequantizeTensor --- */

/* mlxaffine.go:178-208: out = scale*float32(code) + bias, two rounded f32 ops. */
int lthn_o_dequantize(const uint8_t *packed, const uint16_t *scales, const uint16_t *biases,
                      long out_dim, long in_dim, int bits, int gs, float *out) {
    if (!supported_bits(bits)) return LTHN_O_EINVAL;
    if (out_dim <= 0 || in_dim <= 0 || gs <= 0 || in_dim % gs != 0) return LTHN_O_EINVAL;
    int epw = 32 / bits;
    long wpr = in_dim * bits / 32, gpr = in_dim / gs;
    uint32_t mask = (1u << bits) - 1u;
    const uint32_t *words = (const uint32_t *)packed;
#pragma omp parallel for schedule(static)
    for (long r = 0; r < out_dim; r++) {
        for (long j = 0; j < in_dim; j++) {
            uint32_t code = (words[r * wpr + j / epw] >> ((j % epw) * bits)) & mask;
            float scale = lthn_o_bf16_to_f32(scales[r * gpr + j / gs]);
            float bias = lthn_o_bf16_to_f32(biases[r * gpr + j / gs]);
            out[r * in_dim + j] = scale * (float)code + bias;
        }
    }
    return LTHN_O_OK;
}

/* ------------------------------------- a4: ReferenceAffineMatVec (f64) --- */

/* enginetest/quant_reference.go:41-53 affineExtractCode: LSB-first across bytes. */
static uint32_t affine_extract_code(const uint8_t *p, long bit_off, int bits) {
    uint32_t v = 0;
    for (int got = 0; got < bits;) {
        long bi = (bit_off + got) / 8;
        int off = (int)((bit_off + got) % 8);
        int take = 8 - off < bits - got ? 8 - off : bits - got;
        uint32_t chunk = ((uint32_t)p[bi] >> off) & ((1u << take) - 1u);
        v |= chunk << got;
        got += take;
    }
    return v;
}

/* enginetest/quant_reference.go:57-68 affineSetCode (fixture builder). */
void lthn_o_affine_set_code(uint8_t *p, long bit_off, int bits, uint32_t code) {
    for (int got = 0; got < bits;) {
        long bi = (bit_off + got) / 8;
        int off = (int)((bit_off + got) % 8);
        int take = 8 - off < bits - got ? 8 - off : bits - got;
        uint8_t mask = (uint8_t)(((1u << take) - 1u) << off);
        uint8_t shifted = (uint8_t)((code >> got) << off);
        p[bi] = (uint8_t)((p[bi] & ~mask) | (shifted & mask));
        got += take;
    }
}

uint32_t lthn_o_affine_extract_code(const uint8_t *p, long bit_off, int bits) {
    return affine_extract_code(p, bit_off, bits);
}

/* enginetest/quant_reference.go:79-127. bf16 x in, bf16 out, f64 serial sum.
 * Lengths are passed so the reference's validation surface is reproduced. */
int lthn_o_ref_affine_matvec(const uint8_t *x, long x_len, const uint8_t *packed, long packed_len,
                             const uint8_t *scales, long scales_len, const uint8_t *biases, long biases_len,
                             long out_dim, long in_dim, int gs, int bits, uint8_t *out) {
    if (out_dim < 0 || in_dim < 0) return LTHN_O_EINVAL;
    if (out_dim == 0 || in_dim == 0) { if (out_dim > 0) memset(out, 0, (size_t)out_dim * 2); return LTHN_O_OK; }
    if (bits <= 0 || bits > 8) return LTHN_O_EINVAL;
    if (gs <= 0 || in_dim % gs != 0) return LTHN_O_EINVAL;
    if (in_dim * bits % 8 != 0) return LTHN_O_EINVAL;
    if (x_len != in_dim * 2) return LTHN_O_EINVAL;
    long row_packed = in_dim * bits / 8, row_sb = (in_dim / gs) * 2;
    if (packed_len != out_dim * row_packed || scales_len != out_dim * row_sb || biases_len != out_dim * row_sb)
        return LTHN_O_EINVAL;
    double *xf = (double *)malloc(sizeof(double) * (size_t)in_dim);
    const uint16_t *xh = (const uint16_t *)x;
    for (long i = 0; i < in_dim; i++) xf[i] = (double)lthn_o_bf16_to_f32(xh[i]);
    const uint16_t *sh = (const uint16_t *)scales, *bh = (const uint16_t *)biases;
    uint16_t *oh = (uint16_t *)out;
    long gpr = in_dim / gs;
#pragma omp parallel for schedule(static)
    for (long r = 0; r < out_dim; r++) {
        const uint8_t *prow = packed + r * row_packed;
        double acc = 0;
        for (long c = 0; c < in_dim; c++) {
            long g = c / gs;
            float scale = lthn_o_bf16_to_f32(sh[r * gpr + g]);
            float bias = lthn_o_bf16_to_f32(bh[r * gpr + g]);
            uint32_t code = affine_extract_code(prow, c * bits, bits);
            double w = (double)scale * (double)code + (double)bias;
            acc += w * xf[c];
        }
        oh[r] = lthn_o_f32_to_bf16((float)acc);
    }
    free(xf);
    return LTHN_O_OK;
}

/* --------------------- a5: hipReferenceMLXAffineProjection (f32 serial) --- */

/* engine/hip/hip_projection_reference.go:200-222 hipMLXAffineUnpackValue */
static inline uint32_t hip_unpack(const uint32_t *row, long col, int bits) {
    uint64_t bit_off = (uint64_t)col * (uint64_t)bits;
    long wi = (long)(bit_off / 32);
    unsigned shift = (unsigned)(bit_off % 32);
    uint32_t value = row[wi] >> shift;
    if (shift + (unsigned)bits > 32) value |= row[wi + 1] << (32 - shift);
    return value & ((1u << bits) - 1u);
}

/* engine/hip/hip_projection_reference.go:92-116 (+ shape validation :122-145).
 * weight = float32(q)*scale + bias; sum += input[col]*weight, f32, ascending. */
int lthn_o_hip_affine_projection(const float *input, const uint32_t *weights, const uint16_t *scales,
                                 const uint16_t *biases, long rows, long cols, int gs, int bits, float *output) {
    if (bits == 0) bits = 4;
    if (!(bits == 4 || bits == 6 || bits == 8)) return LTHN_O_EINVAL;
    if (rows <= 0 || cols <= 0 || gs <= 0) return LTHN_O_EINVAL;
    if (((uint64_t)cols * (uint64_t)bits) % 32 != 0) return LTHN_O_EINVAL;
    if (cols % gs != 0) return LTHN_O_EINVAL;
    long ppr = cols * bits / 32, gpr = cols / gs;
#pragma omp parallel for schedule(static)
    for (long row = 0; row < rows; row++) {
        const uint32_t *wr = weights + row * ppr;
        float sum = 0;
        for (long col = 0; col < cols; col++) {
            uint32_t q = hip_unpack(wr, col, bits);
            long group = row * gpr + col / gs;
            float weight = (float)q * lthn_o_bf16_to_f32(scales[group]) + lthn_o_bf16_to_f32(biases[group]);
            sum += input[col] * weight;
        }
        output[row] = sum;
    }
    return LTHN_O_OK;
}

/* Batched form of the same arithmetic for `tokens` activation rows
 * (hip_gemma4_q4_oracle_test.go:963-979 hipOracleReferenceProjectionRows calls
 * the projection once per token row). Each (token,row) sum is the identical
 * serial f32 chain; tokens are the inner loop so the compiler can keep several
 * independent chains in flight. x: [tokens, cols], out: [tokens, rows]. */
int lthn_o_hip_affine_projection_rows(const float *x, long tokens, const uint32_t *weights,
                                      const uint16_t *scales, const uint16_t *biases, long rows, long cols,
                                      int gs, int bits, float *out) {
    if (bits == 0) bits = 4;
    if (!(bits == 4 || bits == 6 || bits == 8)) return LTHN_O_EINVAL;
    if (rows <= 0 || cols <= 0 || gs <= 0 || tokens <= 0) return LTHN_O_EINVAL;
    if (((uint64_t)cols * (uint64_t)bits) % 32 != 0 || cols % gs != 0) return LTHN_O_EINVAL;
    long ppr = cols * bits / 32, gpr = cols / gs;
    /* transpose x so the token index is contiguous for each column */
    float *xt = (float *)malloc(sizeof(float) * (size_t)tokens * (size_t)cols);
    for (long t = 0; t < tokens; t++)
        for (long c = 0; c < cols; c++) xt[c * tokens + t] = x[t * cols + c];
#pragma omp parallel
    {
        float *sum = (float *)malloc(sizeof(float) * (size_t)tokens);
#pragma omp for schedule(static)
        for (long row = 0; row < rows; row++) {
            const uint32_t *wr = weights + row * ppr;
            for (long t = 0; t < tokens; t++) sum[t] = 0;
            for (long col = 0; col < cols; col++) {
                uint32_t q = hip_unpack(wr, col, bits);
                long group = row * gpr + col / gs;
                float weight = (float)q * lthn_o_bf16_to_f32(scales[group]) + lthn_o_bf16_to_f32(biases[group]);
                const float *xc = xt + col * tokens;
                for (long t = 0; t < tokens; t++) sum[t] += xc[t] * weight;
            }
            for (long t = 0; t < tokens; t++) out[t * rows + row] = sum[t];
        }
        free(sum);
    }
    free(xt);
    return LTHN_O_OK;
}

/* ---------------------------- a6: attn.matNTQuantHost (timed baseline) --- */

/* model/attn/gated_delta.go:63-89: per output row n dequantise the row with
 * DequantizeTensor (a2), then for every activation row m an f64 dot in ascending
 * k, stored as f32. threads<=1 reproduces the reference's serial loop; threads>1
 * splits the (independent) n loop, per-element arithmetic unchanged. */
int lthn_o_matnt_quant_host(float *out, const float *x, const uint8_t *packed, const uint16_t *scales,
                            const uint16_t *biases, long M, long K, long N, int gs, int bits, int threads) {
    if (!supported_bits(bits) || K <= 0 || gs <= 0 || K % gs != 0 || M < 0 || N < 0) return LTHN_O_EINVAL;
    long wpr = K * bits / 32, gpr = K / gs;
    int nt = threads > 1 ? threads : 1;
#pragma omp parallel num_threads(nt)
    {
        float *wr = (float *)malloc(sizeof(float) * (size_t)K);
#pragma omp for schedule(static)
        for (long n = 0; n < N; n++) {
            int epw = 32 / bits;
            uint32_t mask = (1u << bits) - 1u;
            const uint32_t *words = (const uint32_t *)packed + n * wpr;
            for (long j = 0; j < K; j++) {
                uint32_t code = (words[j / epw] >> ((j % epw) * bits)) & mask;
                float scale = lthn_o_bf16_to_f32(scales[n * gpr + j / gs]);
                float bias = lthn_o_bf16_to_f32(biases[n * gpr + j / gs]);
                wr[j] = scale * (float)code + bias;
            }
            for (long m = 0; m < M; m++) {
                const float *xr = x + m * K;
                double acc = 0;
                for (long k = 0; k < K; k++) acc += (double)xr[k] * (double)wr[k];
                out[m * N + n] = (float)acc;
            }
        }
        free(wr);
    }
    return LTHN_O_OK;
}

/* model/mat.go:12-24 MatNT: out[M,N] = in[M,K]·w[N,K]^T, f64 accumulate. */
void lthn_o_matnt(const float *in, const float *w, long M, long K, long N, float *out) {
#pragma omp parallel for schedule(static)
    for (long n = 0; n < N; n++)
        for (long m = 0; m < M; m++) {
            double acc = 0;
            for (long k = 0; k < K; k++) acc += (double)in[m * K + k] * (double)w[n * K + k];
            out[m * N + n] = (float)acc;
        }
}

/* Prefill matmul as the reference's Metal engine defines it
 * (engine/metal/quant_seam_backend.go:84-110 routes M>1 to MLX affine_qmm_t with
 * bf16 activations, bf16 output; the kernel body lives in ml-explore/mlx v0.32.0,
 * which is not vendored, so its exact reduction order is unpinned): each weight is
 * dequantised as in a2 and rounded to bf16, products are accumulated in f64, and
 * the result is rounded once to bf16. x_bf16: [M,K]; out_bf16: [M,N]. */
int lthn_o_qmm_bf16(const uint16_t *x, const uint8_t *packed, const uint16_t *scales, const uint16_t *biases,
                    long M, long K, long N, int gs, int bits, uint16_t *out) {
    if (!supported_bits(bits) || K <= 0 || gs <= 0 || K % gs != 0 || M < 0 || N < 0) return LTHN_O_EINVAL;
    long wpr = K * bits / 32, gpr = K / gs;
    int epw = 32 / bits;
    uint32_t mask = (1u << bits) - 1u;
#pragma omp parallel
    {
        float *wr = (float *)malloc(sizeof(float) * (size_t)K);
#pragma omp for schedule(static)
        for (long n = 0; n < N; n++) {
            const uint32_t *words = (const uint32_t *)packed + n * wpr;
            for (long j = 0; j < K; j++) {
                uint32_t code = (words[j / epw] >> ((j % epw) * bits)) & mask;
                float scale = lthn_o_bf16_to_f32(scales[n * gpr + j / gs]);
                float bias = lthn_o_bf16_to_f32(biases[n * gpr + j / gs]);
                wr[j] = lthn_o_bf16_to_f32(lthn_o_f32_to_bf16(scale * (float)code + bias));
            }
            for (long m = 0; m < M; m++) {
                const uint16_t *xr = x + m * K;
                double acc = 0;
                for (long k = 0; k < K; k++) acc += (double)lthn_o_bf16_to_f32(xr[k]) * (double)wr[k];
                out[m * N + n] = lthn_o_f32_to_bf16((float)acc);
            }
        }
        free(wr);
    }
    return LTHN_O_OK;
}

/* The same contract with f32 activations in (rounded to bf16 here) and the f64 sums returned as
 * f32 without an output rounding: what a prefill projection computes when the caller keeps its
 * outputs in f32. x: [tokens, cols] f32; out: [tokens, rows] f32. */
int lthn_o_proj_bf16_contract(const float *x, long tokens, const uint32_t *weights, const uint16_t *scales,
                              const uint16_t *biases, long rows, long cols, int gs, int bits, float *out) {
    if (!supported_bits(bits) || cols <= 0 || gs <= 0 || cols % gs != 0 || tokens <= 0 || rows <= 0) return LTHN_O_EINVAL;
    long wpr = cols * bits / 32, gpr = cols / gs;
    int epw = 32 / bits;
    uint32_t mask = (1u << bits) - 1u;
    float *xb = (float *)malloc(sizeof(float) * (size_t)tokens * (size_t)cols);
    for (long i = 0; i < tokens * cols; i++) xb[i] = lthn_o_bf16_to_f32(lthn_o_f32_to_bf16(x[i]));
#pragma omp parallel
    {
        float *wr = (float *)malloc(sizeof(float) * (size_t)cols);
#pragma omp for schedule(static)
        for (long n = 0; n < rows; n++) {
            const uint32_t *words = weights + n * wpr;
            for (long j = 0; j < cols; j++) {
                uint32_t code = (words[j / epw] >> ((j % epw) * bits)) & mask;
                float scale = lthn_o_bf16_to_f32(scales[n * gpr + j / gs]);
                float bias = lthn_o_bf16_to_f32(biases[n * gpr + j / gs]);
                wr[j] = lthn_o_bf16_to_f32(lthn_o_f32_to_bf16(scale * (float)code + bias));
            }
            for (long m = 0; m < tokens; m++) {
                const float *xr = xb + m * cols;
                double acc = 0;
                for (long k = 0; k < cols; k++) acc += (double)xr[k] * (double)wr[k];
                out[m * rows + n] = (float)acc;
            }
        }
        free(wr);
    }
    free(xb);
    return LTHN_O_OK;
}

/* -------------------------------------- a13: RMSNorm / RoPE references --- */

/* engine/hip/hip_transformer_reference.go:171-194 hipReferenceRMSNorm:
 * sumSquares f64 of float32(value*value); rms = float32(sqrt(ss/n + eps));
 * out = value / rms * weight (f32, left to right). */
int lthn_o_rmsnorm(const float *input, const float *weight, long n, float eps, float *out) {
    if (n <= 0 || eps < 0 || isnan(eps) || isinf(eps)) return LTHN_O_EINVAL;
    double ss = 0;
    for (long i = 0; i < n; i++) { float sq = input[i] * input[i]; ss += (double)sq; }
    float rms = (float)sqrt(ss / (double)n + (double)eps);
    if (rms == 0) return LTHN_O_EINVAL;
    for (long i = 0; i < n; i++) out[i] = input[i] / rms * weight[i];
    return LTHN_O_OK;
}

/* hip_transformer_reference.go:242-289 hipReferenceRoPENeoXWithFrequencyDimScale:
 * pairs (i, i+len/2); the first rotary/2 pairs rotate by angle
 * pos * base^(-2i/freq_dim) * freq_scale, f64 trig, cos/sin rounded to f32. */
int lthn_o_rope_neox(const float *input, long n, long position, double base, long freq_dim, long rotary,
                     double freq_scale, float *out) {
    if (n <= 0 || n % 2 != 0 || position < 0 || !(base > 0) || !(freq_scale > 0)) return LTHN_O_EINVAL;
    if (freq_dim < 0 || (freq_dim > 0 && freq_dim < n)) return LTHN_O_EINVAL;
    if (rotary < 0 || rotary > n || rotary % 2 != 0) return LTHN_O_EINVAL;
    if (freq_dim == 0) freq_dim = n;
    if (rotary == 0) rotary = n;
    long half = n / 2, active = rotary / 2;
    for (long pair = 0; pair < half; pair++) {
        long first = pair, second = pair + half;
        if (pair >= active) { out[first] = input[first]; out[second] = input[second]; continue; }
        double frequency = 1 / pow(base, (double)(pair * 2) / (double)freq_dim);
        double angle = (double)position * frequency * freq_scale;
        float c = (float)cos(angle), s = (float)sin(angle);
        float x = input[first], y = input[second];
        out[first] = x * c - y * s;
        out[second] = x * s + y * c;
    }
    return LTHN_O_OK;
}

/* hip_transformer_reference.go:204-240 hipReferenceRoPEWithFrequencyDimScale:
 * interleaved pairs (i, i+1). */
int lthn_o_rope_interleaved(const float *input, long n, long position, double base, long freq_dim,
                            double freq_scale, float *out) {
    if (n <= 0 || n % 2 != 0 || position < 0 || !(base > 0) || !(freq_scale > 0)) return LTHN_O_EINVAL;
    if (freq_dim < 0 || (freq_dim > 0 && freq_dim < n)) return LTHN_O_EINVAL;
    if (freq_dim == 0) freq_dim = n;
    for (long i = 0; i < n; i += 2) {
        double frequency = 1 / pow(base, (double)i / (double)freq_dim);
        double angle = (double)position * frequency * freq_scale;
        float c = (float)cos(angle), s = (float)sin(angle);
        float x = input[i], y = input[i + 1];
        out[i] = x * c - y * s;
        out[i + 1] = x * s + y * c;
    }
    return LTHN_O_OK;
}

/* engine/metal/kernels/norms/lthn_qknorm_rope_bf16.metal:28-110: bf16 in/out,
 * normed = bf16(w * bf16(x*inv)), NeoX pairs (i, i+rotary/2) over the first
 * `rotary` dims, inv_freq = exp2(-(i/(rotary/2)) * log2(theta)), tail passes
 * through. Trig here is libm cosf/sinf where the shader uses Metal's fast
 * variants, so device agreement is to tolerance, not bit-exact. */
int lthn_o_qknorm_rope_bf16(const uint16_t *x, const uint16_t *w, long heads, long head_dim, long rotary,
                            float eps, float scale, long position, float log2_theta, uint16_t *out) {
    if (heads <= 0 || head_dim <= 0 || head_dim > 512 || rotary < 0 || rotary > head_dim || rotary % 2) return LTHN_O_EINVAL;
    for (long h = 0; h < heads; h++) {
        const uint16_t *xh = x + h * head_dim;
        float acc = 0;
        for (long d = 0; d < head_dim; d++) { float xi = lthn_o_bf16_to_f32(xh[d]); acc += xi * xi; }
        float inv = 1.0f / sqrtf(acc / (float)head_dim + eps);
        float normed[512];
        for (long d = 0; d < head_dim; d++) {
            float inner = lthn_o_bf16_to_f32(lthn_o_f32_to_bf16(lthn_o_bf16_to_f32(xh[d]) * inv));
            normed[d] = lthn_o_bf16_to_f32(lthn_o_f32_to_bf16(lthn_o_bf16_to_f32(w[d]) * inner));
        }
        long hrot = rotary / 2;
        for (long d = 0; d < head_dim; d++) {
            if (d >= rotary) { out[h * head_dim + d] = lthn_o_f32_to_bf16(normed[d]); continue; }
            long i = d < hrot ? d : d - hrot;
            float dfrac = (float)i / (float)hrot;
            float inv_freq = exp2f(-dfrac * log2_theta);
            float theta = scale * (float)position * inv_freq;
            float c = cosf(theta), s = sinf(theta);
            float x1 = normed[i], x2 = normed[i + hrot];
            out[h * head_dim + d] = lthn_o_f32_to_bf16(d < hrot ? x1 * c - x2 * s : x1 * s + x2 * c);
        }
    }
    return LTHN_O_OK;
}

/* ------------------------------------------- a14: attention reference ---- */

/* engine/hip/moe_quant_reference.go:268-286 softmaxFloat32 (in place into out) */
static void softmax_f32(const float *values, long n, float *out) {
    float maxv = values[0];
    for (long i = 1; i < n; i++) if (values[i] > maxv) maxv = values[i];
    double sum = 0;
    for (long i = 0; i < n; i++) { double e = exp((double)(values[i] - maxv)); out[i] = (float)e; sum += e; }
    for (long i = 0; i < n; i++) out[i] = (float)((double)out[i] / sum);
}

/* hip_transformer_reference.go:295-330 hipReferenceSingleHeadAttentionWithScale.
 * keys/values are `count` rows, `stride` floats apart (so a [pos, kvHeads*dim]
 * cache can be addressed in place); scale 0 means 1/sqrt(dim). */
int lthn_o_attention_single_head(const float *query, const float *keys, const float *values, long count,
                                 long dim, long stride, float scale, float *out, float *weights_scratch) {
    if (dim <= 0 || count <= 0 || scale < 0 || isnan(scale) || isinf(scale)) return LTHN_O_EINVAL;
    if (scale == 0) scale = (float)(1 / sqrt((double)dim));
    float *scores = weights_scratch;
    for (long i = 0; i < count; i++) {
        const float *key = keys + i * stride;
        float score = 0;
        for (long j = 0; j < dim; j++) score += query[j] * key[j];
        scores[i] = score * scale;
    }
    softmax_f32(scores, count, scores);
    for (long j = 0; j < dim; j++) out[j] = 0;
    for (long i = 0; i < count; i++) {
        const float *value = values + i * stride;
        for (long j = 0; j < dim; j++) out[j] += scores[i] * value[j];
    }
    return LTHN_O_OK;
}

/* hip_gemma4_q4_oracle_test.go:1085-1101 rocmOracleKVHeadForQuery */
long lthn_o_kv_head_for_query(long query_head, long query_heads, long kv_heads) {
    if (kv_heads <= 1 || query_heads <= kv_heads) return kv_heads <= 1 ? 0 : query_head;
    long group = query_heads / kv_heads;
    if (group == 0) return 0;
    long kv = query_head / group;
    return kv >= kv_heads ? kv_heads - 1 : kv;
}

/* ------------------------------------------------ GELU, greedy, embed ---- */

/* engine/hip/hip_gemma4_q4_layer.go:3582-3597 hipGemma4Q4HostGELU (tanh form, f64) */
void lthn_o_gelu_tanh(const float *input, long n, float *out) {
    const double sqrt2_over_pi = 0.7978845608028654, coeff = 0.044715;
    for (long i = 0; i < n; i++) {
        double x = (double)input[i];
        out[i] = (float)(0.5 * x * (1 + tanh(sqrt2_over_pi * (x + coeff * x * x * x))));
    }
}

/* hip_transformer_reference.go:400-414 hipReferenceGreedySample: strict >, so the
 * lowest index wins ties (same rule as model/sample.go:33-50 on bf16 logits). */
long lthn_o_greedy_f32(const float *logits, long n) {
    if (n <= 0) return -1;
    long index = 0; float value = logits[0];
    for (long i = 1; i < n; i++) if (logits[i] > value) { index = i; value = logits[i]; }
    return index;
}

/* model/sample.go:29-50 Greedy over bf16 logits, best starts at -Inf, strict >. */
long lthn_o_greedy_bf16(const uint16_t *logits, long vocab) {
    long best = -1; float best_v = -INFINITY;
    for (long i = 0; i < vocab; i++) {
        float v = lthn_o_bf16_to_f32(logits[i]);
        if (v > best_v) { best = i; best_v = v; }
    }
    return best;
}

/* hip_transformer_reference.go:60-92 hipReferenceMLXAffineEmbeddingLookup (one id) */
int lthn_o_affine_embedding_row(const uint32_t *weights, const uint16_t *scales, const uint16_t *biases,
                                long vocab, long hidden, int gs, int bits, long id, float *out) {
    if (bits == 0) bits = 4;
    if (id < 0 || id >= vocab || hidden % gs != 0) return LTHN_O_EINVAL;
    long ppr = hidden * bits / 32, gpr = hidden / gs;
    for (long dim = 0; dim < hidden; dim++) {
        uint32_t q = hip_unpack(weights + id * ppr, dim, bits);
        long group = id * gpr + dim / gs;
        out[dim] = (float)q * lthn_o_bf16_to_f32(scales[group]) + lthn_o_bf16_to_f32(biases[group]);
    }
    return LTHN_O_OK;
}

/* model/norm_bias.go:22-49 foldNormBiasOne for f32 weights: w+1 in f32. */
void lthn_o_fold_norm_bias_one_f32(const float *w, long n, float *out) {
    for (long i = 0; i < n; i++) out[i] = w[i] + 1;
}
/* same file, bf16 branch: f32(bf16)+1 rounded RNE to bf16. */
void lthn_o_fold_norm_bias_one_bf16(const uint16_t *w, long n, uint16_t *out) {
    for (long i = 0; i < n; i++) out[i] = lthn_o_f32_to_bf16(lthn_o_bf16_to_f32(w[i]) + 1);
}

/* --------------------------------------------- synthetic weight source --- */

/* Counter-based generator used to fill benchmark-sized synthetic tensors with
 * approximately N(0, sigma) values identically on CPU and GPU (integer hashing
 * plus one f32 multiply, so both sides agree bit for bit). It is this build's
 * own construction, not part of the reference: the reference benchmarks on
 * downloaded checkpoints. Value = sigma * (sum of eight 16-bit uniforms - mean)
 * / stddev of that sum (Irwin-Hall, n=8). */
static inline uint64_t splitmix64(uint64_t z) {
    z += 0x9e3779b97f4a7c15ull;
    z = (z ^ (z >> 30)) * 0xbf58476d1ce4e5b9ull;
    z = (z ^ (z >> 27)) * 0x94d049bb133111ebull;
    return z ^ (z >> 31);
}
float lthn_o_synth_normal(uint64_t seed, uint64_t index, float sigma) {
    uint64_t a = splitmix64(seed * 0xd1342543de82ef95ull + 2 * index);
    uint64_t b = splitmix64(seed * 0xd1342543de82ef95ull + 2 * index + 1);
    int32_t s = 0;
    for (int i = 0; i < 4; i++) { s += (int32_t)((a >> (16 * i)) & 0xffff); s += (int32_t)((b >> (16 * i)) & 0xffff); }
    /* mean = 8*65535/2 = 262140; var = 8*(65536^2-1)/12 -> std = 53509.0305... */
    float centered = (float)(s - 262140);
    return centered * (sigma * (1.0f / 53509.03f));
}
void lthn_o_synth_normal_fill(uint64_t seed, uint64_t first, long n, float sigma, float *out) {
    float k = sigma * (1.0f / 53509.03f);
#pragma omp parallel for schedule(static)
    for (long i = 0; i < n; i++) {
        uint64_t idx = first + (uint64_t)i;
        uint64_t a = splitmix64(seed * 0xd1342543de82ef95ull + 2 * idx);
        uint64_t b = splitmix64(seed * 0xd1342543de82ef95ull + 2 * idx + 1);
        int32_t s = 0;
        for (int j = 0; j < 4; j++) { s += (int32_t)((a >> (16 * j)) & 0xffff); s += (int32_t)((b >> (16 * j)) & 0xffff); }
        out[i] = (float)(s - 262140) * k;
    }
}
