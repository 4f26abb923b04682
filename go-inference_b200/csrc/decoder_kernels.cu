// decoder_kernels.cu — the small fused kernels around the quantized linears of a
// Gemma-style decoder step: embedding row dequantise, RMSNorm (+residual, +next
// norm), per-head RMSNorm + NeoX RoPE + KV append, split-KV decode attention over
// the seq-major bf16 cache, and greedy argmax.
//
// They are all latency-sized (a few KB to a few MB per launch); the design goal is
// few launches and exact, reproducible arithmetic:
//  * sums of squares are accumulated in f64 so the reciprocal RMS is the same
//    value the CPU reference computes (hipReferenceRMSNorm, engine/hip/
//    hip_transformer_reference.go:171-194), and x / rms * w is issued as separately
//    rounded f32 operations;
//  * RoPE uses a cos/sin table computed on the host in f64 exactly as the reference
//    does (hip_transformer_reference.go:242-289), so the rotation is bit-identical;
//  * reductions have a fixed order (no atomics in the value path).
#include "common.cuh"
#include "decoder_kernels.hpp"
#include <algorithm>
#include <cstdlib>
#include "attn_item.cuh"

namespace lthn {

// ---- block reductions ---------------------------------------------------------------
__device__ __forceinline__ double block_sum_f64(double v, double* sh) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    __syncthreads();
    if (lane == 0) sh[warp] = v;
    __syncthreads();
    double t = 0.0;
    for (int w = 0; w < nw; w++) t += sh[w];
    return t;
}

// ---- embedding ----------------------------------------------------------------------
// h[row, :] = (float(code)*scale + bias) * embed_scale for token ids[row]
// (hipReferenceMLXAffineEmbeddingLookup, hip_transformer_reference.go:60-92, and the
// output scale of engine/hip/kernels/embedding/lookup.hipinc:3-31).
__global__ void embed_kernel(const int32_t* __restrict__ ids, const uint32_t* __restrict__ packed,
                             const uint16_t* __restrict__ scales, const uint16_t* __restrict__ biases, int hidden,
                             int vocab, float embed_scale, float* __restrict__ out) {
    pdl_trigger();
    pdl_wait();
    const int row = blockIdx.x;
    int id = ids[row];
    if (id < 0 || id >= vocab) id = 0;  // ids are validated on the host; stay in bounds regardless
    const int wpr = hidden >> 3, gpr = hidden >> 6;
    for (int w = threadIdx.x; w < wpr; w += blockDim.x) {
        const uint32_t word = __ldg(packed + (int64_t)id * wpr + w);
        const int g = w >> 3;
        const float s = bf16_bits_to_f32(__ldg(scales + (int64_t)id * gpr + g));
        const float b = bf16_bits_to_f32(__ldg(biases + (int64_t)id * gpr + g));
        float* o = out + (int64_t)row * hidden + w * 8;
#pragma unroll
        for (int p = 0; p < 8; p++) {
            const float q = (float)((word >> (4 * p)) & 15u);
            o[p] = __fmul_rn(__fadd_rn(__fmul_rn(q, s), b), embed_scale);
        }
    }
}

// ---- RMSNorm family -------------------------------------------------------------------
// mode 0: out = norm(x, w)
// mode 1: h = h + norm(a, w_post); out = norm(h, w_next)      (post-norm, residual, next pre-norm)
// One CTA per row. (hipOracleReferenceLayer, hip_gemma4_q4_oracle_test.go:925-951.)
// cols/split (optional): the output additionally as bf16 hi/mid/lo columns
// [rows*split, width] (column row*split+j), the form the tensor-core matvec consumes.
__device__ __forceinline__ void store_split(uint16_t* cols, int split, int row, int width, int i, float v) {
    float r = v;
    for (int j = 0; j < split; j++) {
        const uint16_t hbits = f32_to_bf16_bits(r);
        cols[((int64_t)row * split + j) * width + i] = hbits;
        r -= bf16_bits_to_f32(hbits);
    }
}

__global__ void __launch_bounds__(1024) rmsnorm_kernel(const float* __restrict__ a, float* __restrict__ h,
                                                      const float* __restrict__ w_post,
                                                      const float* __restrict__ w_next, float* __restrict__ out,
                                                      int width, float eps, int mode, uint16_t* __restrict__ cols,
                                                      int split) {
    pdl_trigger();
    pdl_wait();
    __shared__ double sh[32];
    const int row = blockIdx.x;
    const float* ar = a + (int64_t)row * width;
    float* hr = h ? h + (int64_t)row * width : nullptr;
    float* orow = out ? out + (int64_t)row * width : nullptr;  // the f32 output is optional when cols is given
    double ss = 0.0;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        const float v = ar[i];
        ss += (double)__fmul_rn(v, v);
    }
    ss = block_sum_f64(ss, sh);
    const float rms = (float)sqrt(ss / (double)width + (double)eps);
    if (mode == 0) {
        for (int i = threadIdx.x; i < width; i += blockDim.x) {
            const float v = __fmul_rn(__fdiv_rn(ar[i], rms), w_post[i]);
            if (orow) orow[i] = v;
            if (cols) store_split(cols, split, row, width, i, v);
        }
        return;
    }
    double ss2 = 0.0;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        const float n = __fmul_rn(__fdiv_rn(ar[i], rms), w_post[i]);
        const float v = __fadd_rn(hr[i], n);
        hr[i] = v;
        ss2 += (double)__fmul_rn(v, v);
    }
    ss2 = block_sum_f64(ss2, sh);
    const float rms2 = (float)sqrt(ss2 / (double)width + (double)eps);
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        const float v = __fmul_rn(__fdiv_rn(hr[i], rms2), w_next[i]);
        if (orow) orow[i] = v;
        if (cols) store_split(cols, split, row, width, i, v);
    }
}

// Same arithmetic with the row held in registers (up to 8 elements per thread): every
// global load (activation, residual, both weight vectors) is issued before the first
// reduction, so the kernel costs one memory round trip instead of three.
__global__ void __launch_bounds__(1024) rmsnorm_reg_kernel(const float* __restrict__ a, float* __restrict__ h,
                                                          const float* __restrict__ w_post,
                                                          const float* __restrict__ w_next, float* __restrict__ out,
                                                          int width, float eps, int mode, uint16_t* __restrict__ cols,
                                                          int split) {
    pdl_trigger();
    pdl_wait();
    constexpr int MAXE = 8;
    __shared__ double sh[32];
    const int row = blockIdx.x;
    const float* ar = a + (int64_t)row * width;
    float* hr = h ? h + (int64_t)row * width : nullptr;
    float* orow = out ? out + (int64_t)row * width : nullptr;  // optional when cols is given
    float av[MAXE], hv[MAXE], wp[MAXE], wn[MAXE];
#pragma unroll
    for (int k = 0; k < MAXE; k++) {
        const int i = threadIdx.x + k * blockDim.x;
        av[k] = 0.f; hv[k] = 0.f; wp[k] = 0.f; wn[k] = 0.f;
        if (i < width) {
            av[k] = ar[i];
            wp[k] = w_post[i];
            if (mode) { hv[k] = hr[i]; wn[k] = w_next[i]; }
        }
    }
    double ss = 0.0;
#pragma unroll
    for (int k = 0; k < MAXE; k++) ss += (double)__fmul_rn(av[k], av[k]);
    ss = block_sum_f64(ss, sh);
    const float rms = (float)sqrt(ss / (double)width + (double)eps);
    double ss2 = 0.0;
#pragma unroll
    for (int k = 0; k < MAXE; k++) {
        const int i = threadIdx.x + k * blockDim.x;
        if (i >= width) continue;
        const float n = __fmul_rn(__fdiv_rn(av[k], rms), wp[k]);
        if (mode == 0) {
            if (orow) orow[i] = n;
            if (cols) store_split(cols, split, row, width, i, n);
        } else {
            hv[k] = __fadd_rn(hv[k], n);
            hr[i] = hv[k];
            ss2 += (double)__fmul_rn(hv[k], hv[k]);
        }
    }
    if (mode == 0) return;
    ss2 = block_sum_f64(ss2, sh);
    const float rms2 = (float)sqrt(ss2 / (double)width + (double)eps);
#pragma unroll
    for (int k = 0; k < MAXE; k++) {
        const int i = threadIdx.x + k * blockDim.x;
        if (i >= width) continue;
        const float v = __fmul_rn(__fdiv_rn(hv[k], rms2), wn[k]);
        if (orow) orow[i] = v;
        if (cols) store_split(cols, split, row, width, i, v);
    }
}

// The same arithmetic for many rows at once (prefill chunks): one warp per row, shuffles only, no
// block barrier. The row (a few KB) is read three times from L1/L2 instead of being held in
// registers, so any width is served; sums of squares stay f64 as above.
__global__ void __launch_bounds__(128) rmsnorm_rows_kernel(const float* __restrict__ a, float* __restrict__ h,
                                                          const float* __restrict__ w_post,
                                                          const float* __restrict__ w_next, float* __restrict__ out,
                                                          int rows, int width, float eps, int mode,
                                                          uint16_t* __restrict__ cols, int split) {
    pdl_trigger();
    pdl_wait();
    const int lane = threadIdx.x & 31;
    const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= rows) return;
    const float* ar = a + (int64_t)row * width;
    float* hr = h ? h + (int64_t)row * width : nullptr;
    float* orow = out ? out + (int64_t)row * width : nullptr;
    const int w4 = width >> 2;  // width is a multiple of 4 (checked by the launcher)
    double ss = 0.0;
    for (int i = lane; i < w4; i += 32) {
        const float4 v = ((const float4*)ar)[i];
        ss += (double)__fmul_rn(v.x, v.x) + (double)__fmul_rn(v.y, v.y) + (double)__fmul_rn(v.z, v.z) + (double)__fmul_rn(v.w, v.w);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    const float rms = (float)sqrt(ss / (double)width + (double)eps);
    auto emit = [&](int i, float4 v) {
        if (orow) ((float4*)orow)[i] = v;
        if (cols) {
            const float e[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int k = 0; k < 4; k++) store_split(cols, split, row, width, 4 * i + k, e[k]);
        }
    };
    if (mode == 0) {
        for (int i = lane; i < w4; i += 32) {
            const float4 v = ((const float4*)ar)[i], w = ((const float4*)w_post)[i];
            emit(i, make_float4(__fmul_rn(__fdiv_rn(v.x, rms), w.x), __fmul_rn(__fdiv_rn(v.y, rms), w.y),
                                __fmul_rn(__fdiv_rn(v.z, rms), w.z), __fmul_rn(__fdiv_rn(v.w, rms), w.w)));
        }
        return;
    }
    double ss2 = 0.0;
    for (int i = lane; i < w4; i += 32) {
        const float4 v = ((const float4*)ar)[i], w = ((const float4*)w_post)[i];
        float4 hv = ((float4*)hr)[i];
        hv.x = __fadd_rn(hv.x, __fmul_rn(__fdiv_rn(v.x, rms), w.x));
        hv.y = __fadd_rn(hv.y, __fmul_rn(__fdiv_rn(v.y, rms), w.y));
        hv.z = __fadd_rn(hv.z, __fmul_rn(__fdiv_rn(v.z, rms), w.z));
        hv.w = __fadd_rn(hv.w, __fmul_rn(__fdiv_rn(v.w, rms), w.w));
        ((float4*)hr)[i] = hv;
        ss2 += (double)__fmul_rn(hv.x, hv.x) + (double)__fmul_rn(hv.y, hv.y) + (double)__fmul_rn(hv.z, hv.z) + (double)__fmul_rn(hv.w, hv.w);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss2 += __shfl_xor_sync(0xffffffffu, ss2, o);
    const float rms2 = (float)sqrt(ss2 / (double)width + (double)eps);
    if (!orow && !cols) return;
    for (int i = lane; i < w4; i += 32) {
        const float4 hv = ((const float4*)hr)[i], w = ((const float4*)w_next)[i];
        emit(i, make_float4(__fmul_rn(__fdiv_rn(hv.x, rms2), w.x), __fmul_rn(__fdiv_rn(hv.y, rms2), w.y),
                            __fmul_rn(__fdiv_rn(hv.z, rms2), w.z), __fmul_rn(__fdiv_rn(hv.w, rms2), w.w)));
    }
}

// ---- tensor-parallel residual RMSNorm over peer memory ---------------------------------
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ float ld_relaxed_sys_f32(const float* p) {
    float v;
    asm volatile("ld.relaxed.sys.global.f32 %0, [%1];" : "=f"(v) : "l"(p) : "memory");
    return v;
}

// Exchange protocol. Every rank runs the same sequence of these kernels; exchange number seq
// (kept in local memory, advanced by the last CTA of each launch) names the current one.
//  1. the projection kernel before this one (same stream) wrote this rank's partial sums into
//     its buffer for this call site; the kernel boundary makes them visible;
//  2. CTA 0 stores seq into element [rank] of every peer's flag array (release, system scope);
//  3. every CTA waits until all t elements of the local flag array are >= seq (acquire), with a
//     bounded number of polls: if a peer never arrives the kernel records status bit 256 and goes
//     on, so that the context stays usable and the host reports the failure;
//  4. partials are read from the peers' buffers and added in rank order, so every rank computes
//     bit-identical sums.
// Buffers are not overwritten early: a rank reuses a call site's buffer only two exchanges later,
// after it has passed the next exchange, which every peer signals only after finishing this one.
__global__ void __launch_bounds__(1024) rmsnorm_gather_kernel(const PeerGather pg, float* __restrict__ h,
                                                             const float* __restrict__ w_post,
                                                             const float* __restrict__ w_next, float* __restrict__ out,
                                                             int width, float eps, uint16_t* __restrict__ cols, int split) {
    pdl_trigger();
    pdl_wait();
    constexpr int MAXE = 8;
    __shared__ double sh[32];
    __shared__ uint32_t seq_s;
    const int row = blockIdx.x;
    if (threadIdx.x == 0) seq_s = *(volatile uint32_t*)&pg.ctr[0] + 1u;
    __syncthreads();
    const uint32_t seq = seq_s;
    if (threadIdx.x < pg.t) {
        if (blockIdx.x == 0) {
            __threadfence_system();
            st_release_sys(pg.flag_out[threadIdx.x] + pg.rank, seq);
        }
        bool ok = false;
        const uint32_t limit = pg.poll_limit ? pg.poll_limit : (1u << 21);
        for (uint32_t it = 0; it < limit; ++it) {
            if ((int32_t)(ld_acquire_sys(pg.flag_in + threadIdx.x) - seq) >= 0) { ok = true; break; }
            __nanosleep(it < 64 ? 20 : 500);
        }
        if (!ok) atomicOr(pg.status, 256u);
    }
    __syncthreads();
    float* hr = h + (int64_t)row * width;
    float* orow = out + (int64_t)row * width;
    float av[MAXE], hv[MAXE], wp[MAXE], wn[MAXE];
#pragma unroll
    for (int k = 0; k < MAXE; k++) {
        const int i = threadIdx.x + k * blockDim.x;
        av[k] = 0.f; hv[k] = 0.f; wp[k] = 0.f; wn[k] = 0.f;
        if (i < width) {
            float pv[8];
#pragma unroll
            for (int r = 0; r < 8; r++) pv[r] = r < pg.t ? ld_relaxed_sys_f32(pg.part[r] + (int64_t)row * width + i) : 0.f;
            float sum = pv[0];
#pragma unroll
            for (int r = 1; r < 8; r++) if (r < pg.t) sum = __fadd_rn(sum, pv[r]);
            av[k] = sum;
            wp[k] = w_post[i]; hv[k] = hr[i]; wn[k] = w_next[i];
        }
    }
    double ss = 0.0;
#pragma unroll
    for (int k = 0; k < MAXE; k++) ss += (double)__fmul_rn(av[k], av[k]);
    ss = block_sum_f64(ss, sh);
    const float rms = (float)sqrt(ss / (double)width + (double)eps);
    double ss2 = 0.0;
#pragma unroll
    for (int k = 0; k < MAXE; k++) {
        const int i = threadIdx.x + k * blockDim.x;
        if (i >= width) continue;
        const float n = __fmul_rn(__fdiv_rn(av[k], rms), wp[k]);
        hv[k] = __fadd_rn(hv[k], n);
        hr[i] = hv[k];
        ss2 += (double)__fmul_rn(hv[k], hv[k]);
    }
    ss2 = block_sum_f64(ss2, sh);
    const float rms2 = (float)sqrt(ss2 / (double)width + (double)eps);
#pragma unroll
    for (int k = 0; k < MAXE; k++) {
        const int i = threadIdx.x + k * blockDim.x;
        if (i >= width) continue;
        const float v = __fmul_rn(__fdiv_rn(hv[k], rms2), wn[k]);
        orow[i] = v;
        if (cols) store_split(cols, split, row, width, i, v);
    }
    // the last CTA to finish advances the sequence number (every CTA read it before arriving)
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        if (atomicAdd(&pg.ctr[1], 1u) == gridDim.x - 1) {
            pg.ctr[1] = 0u;
            __threadfence();
            *(volatile uint32_t*)&pg.ctr[0] = seq;
        }
    }
}

// ---- per-head RMSNorm + NeoX RoPE + KV append -----------------------------------------
// qkv: [rows, (Hq + 2*Hkv) * D] f32 (q heads, then k heads, then v heads).
// q heads -> q_out [rows, Hq*D] f32 (normed, rotated); k heads -> bf16 cache row at the
// token's position; v heads -> bf16 cache row (no norm for this architecture).
// One CTA per (row, head); D/2 threads, thread i owns the rotation pair (i, i + D/2).
// (rocm_rms_norm_rope_heads, engine/hip/kernels/norms/rms_norm.hipinc:306-377;
// lthn_qknorm_rope_bf16, engine/metal/kernels/norms/lthn_qknorm_rope_bf16.metal.)
__global__ void qknorm_rope_append_kernel(const float* __restrict__ qkv, const float* __restrict__ q_norm,
                                          const float* __restrict__ k_norm, const float2* __restrict__ rope_table,
                                          const int32_t* __restrict__ row_pos, const int32_t* __restrict__ row_lane,
                                          float* __restrict__ q_out, uint16_t* __restrict__ kcache,
                                          uint16_t* __restrict__ vcache, int Hq, int Hkv, int D, float eps,
                                          int64_t lane_stride, int max_len, double inv_d) {
    pdl_trigger();
    pdl_wait();
    __shared__ double sh[32];
    const int row = blockIdx.x, head = blockIdx.y, i = threadIdx.x, half = D >> 1;
    const int QKV = (Hq + 2 * Hkv) * D;
    const float* src = qkv + (int64_t)row * QKV + (int64_t)head * D;
    const int pos = row_pos[row];
    const int KR = Hkv * D;
    if (head >= Hq + Hkv) {  // value head: round to bf16 and store
        const int vh = head - Hq - Hkv;
        uint16_t* dst = vcache + (int64_t)row_lane[row] * lane_stride + (int64_t)pos * KR + vh * D;
        dst[i] = f32_to_bf16_bits(src[i]);
        dst[i + half] = f32_to_bf16_bits(src[i + half]);
        return;
    }
    const float x0 = src[i], x1 = src[i + half];
    // the weights and the rotation are loaded before the reduction is waited for; rms and the two divisions take
    // the short forms of the matvec prologues (fast_rms, fast_div: no f64 square root, no branch)
    const float* w = head < Hq ? q_norm : k_norm;
    const float w0 = w[i], w1 = w[i + half];
    const float2 cs = rope_table[(int64_t)min(pos, max_len - 1) * half + i];
    double ss = (double)__fmul_rn(x0, x0) + (double)__fmul_rn(x1, x1);
    ss = block_sum_f64(ss, sh);
    const FastDiv k = fast_div_by(fast_rms(ss, inv_d, eps));
    const float n0 = __fmul_rn(fast_div(x0, k), w0);
    const float n1 = __fmul_rn(fast_div(x1, k), w1);
    const float r0 = __fsub_rn(__fmul_rn(n0, cs.x), __fmul_rn(n1, cs.y));
    const float r1 = __fadd_rn(__fmul_rn(n0, cs.y), __fmul_rn(n1, cs.x));
    if (head < Hq) {
        float* dst = q_out + (int64_t)row * Hq * D + (int64_t)head * D;
        dst[i] = r0;
        dst[i + half] = r1;
    } else {
        const int kh = head - Hq;
        uint16_t* dst = kcache + (int64_t)row_lane[row] * lane_stride + (int64_t)pos * KR + kh * D;
        dst[i] = f32_to_bf16_bits(r0);
        dst[i + half] = f32_to_bf16_bits(r1);
    }
}

// Standalone fused per-head RMSNorm + RoPE on f32 rows (no cache append), for the
// C entry point and its parity test: x [rows, heads*D] -> out, positions per row.
__global__ void rmsnorm_rope_kernel(const float* __restrict__ x, const float* __restrict__ w,
                                    const int32_t* __restrict__ positions, float* __restrict__ out, int heads, int D,
                                    int rotary, float eps, float rope_base, int out_bf16_double_round) {
    __shared__ double sh[32];
    const int row = blockIdx.x, head = blockIdx.y, i = threadIdx.x, half = D >> 1;
    const float* src = x + ((int64_t)row * heads + head) * D;
    const float x0 = src[i], x1 = src[i + half];
    double ss = (double)__fmul_rn(x0, x0) + (double)__fmul_rn(x1, x1);
    ss = block_sum_f64(ss, sh);
    const float rms = (float)sqrt(ss / (double)D + (double)eps);
    float n0, n1;
    if (out_bf16_double_round) {
        // Metal rounding seams: bf16(w * bf16(x * inv)) (lthn_qknorm_rope_bf16.metal:75-78)
        const float inv = 1.0f / sqrtf((float)(ss / (double)D) + eps);
        n0 = bf16_bits_to_f32(f32_to_bf16_bits(w[i] * bf16_bits_to_f32(f32_to_bf16_bits(x0 * inv))));
        n1 = bf16_bits_to_f32(f32_to_bf16_bits(w[i + half] * bf16_bits_to_f32(f32_to_bf16_bits(x1 * inv))));
    } else {
        n0 = __fmul_rn(__fdiv_rn(x0, rms), w[i]);
        n1 = __fmul_rn(__fdiv_rn(x1, rms), w[i + half]);
    }
    float* dst = out + ((int64_t)row * heads + head) * D;
    const int active = rotary >> 1;
    // NeoX pairing is (i, i + D/2); the first rotary/2 pairs rotate
    if (i >= active) { dst[i] = n0; dst[i + half] = n1; return; }
    const double freq = 1.0 / pow((double)rope_base, (double)(2 * i) / (double)D);
    const double angle = (double)positions[row] * freq;
    const float c = (float)cos(angle), s = (float)sin(angle);
    float r0 = __fsub_rn(__fmul_rn(n0, c), __fmul_rn(n1, s));
    float r1 = __fadd_rn(__fmul_rn(n0, s), __fmul_rn(n1, c));
    if (out_bf16_double_round) { r0 = bf16_bits_to_f32(f32_to_bf16_bits(r0)); r1 = bf16_bits_to_f32(f32_to_bf16_bits(r1)); }
    dst[i] = r0;
    dst[i + half] = r1;
}

// ---- decode attention over the seq-major bf16 cache -----------------------------------
// cache layout per lane: [max_len][Hkv*D] bf16 (k_seq_stride = Hkv*D, k_head_stride = D;
// engine/metal/decode_step.go:20-26). One CTA handles one (row, bundle of GQ query heads that
// share a kv head, key chunk), so K and V are streamed once per bundle
// (rocm_attention_heads_chunked_stage1 _gqa variants, engine/hip/kernels/attention/
// chunked.hipinc). Eight lanes share a key position, each holding D/8 of the head dimension;
// a 128-thread CTA covers 16*NIT positions and issues every K and V load of its chunk before
// any arithmetic (the chunk is sized so they fit in registers: 8192/D positions), so a chunk
// costs one memory round trip. Scores stay in registers; the chunk result (max, sum,
// unnormalised accumulator) goes to scratch and is merged by sdpa_merge_kernel (stage 2).
// With a single chunk the normalised output is written directly.
// Two forms. sdpa_decode_kernel: a chunk is one tile (16*NIT positions), the chunk maximum is formed across the
// four warps before any weight is computed; 80-98 registers, five or six CTAs per SM - the form for batched rows
// (16 lanes: 12 % faster per step than the other form, whose registers allow two or three CTAs per SM).
// sdpa_decode_tiles_kernel: a chunk is one or more tiles walked with a running softmax per warp (no block-wide
// barrier before the weights; with several tiles fewer partials for the merge and fewer CTA prologues), at
// 140-206 registers; used for one or two rows, where the grid is small and the chain of one CTA is what counts
// (26-layer model 908 -> 940 tok/s at one tile per chunk, 62-layer model 141.5 -> 146.5 with three).
template <int D, int GQ>
__global__ void __launch_bounds__(128) sdpa_decode_kernel(const SdpaArgs a) {
    pdl_trigger();
    pdl_wait();
    constexpr int E = D / 8;          // elements per lane
    constexpr int V8 = E / 8;         // 16-byte loads per lane per row
    constexpr int NIT = 512 / D > 0 ? 512 / D : 1;  // positions per lane group: 16*NIT per CTA
    __shared__ float red[4][GQ][D + 2];
    __shared__ float smax[GQ][4], ssum[GQ][4];

    // blockIdx.x indexes a bundle of GQ consecutive query heads that share one kv head
    const int row = blockIdx.z, chunk = blockIdx.y;
    const int qh0 = blockIdx.x * GQ, kvh = qh0 / (a.Hq / a.Hkv);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int l8 = lane & 7, pg = warp * 4 + (lane >> 3);  // position group 0..15
    const int ctx = a.row_pos[row] + 1;                    // keys 0..pos inclusive
    const int lo = a.window > 0 ? max(0, ctx - a.window) : 0;  // sliding block: keys lo..pos
    const int p0 = chunk * (16 * NIT);
    if (p0 >= ctx || p0 + 16 * NIT <= lo) return;
    const int KR = a.Hkv * D;
    const uint16_t* kbase = a.kcache + (int64_t)a.row_lane[row] * a.lane_stride + (int64_t)kvh * D;
    const uint16_t* vbase = a.vcache + (int64_t)a.row_lane[row] * a.lane_stride + (int64_t)kvh * D;

    // ---- every load of the chunk goes out first ---------------------------------------------
    uint4 kreg[NIT][V8], vreg[NIT][V8];
    bool valid[NIT];
#pragma unroll
    for (int i = 0; i < NIT; i++) {
        const int p = p0 + pg + 16 * i;
        valid[i] = p < ctx && p >= lo;
        const int64_t off = (int64_t)(valid[i] ? p : min(max(p0, lo), ctx - 1)) * KR;
#pragma unroll
        for (int v = 0; v < V8; v++) {
            kreg[i][v] = __ldg((const uint4*)(kbase + off + (v * 8 + l8) * 8));
            vreg[i][v] = __ldg((const uint4*)(vbase + off + (v * 8 + l8) * 8));
        }
    }
    // query slices of this lane for the GQ heads, pre-multiplied by the softmax scale
    float q[GQ][E];
#pragma unroll
    for (int h = 0; h < GQ; h++) {
        const float* qh = a.q + ((int64_t)row * a.Hq + qh0 + h) * D;
#pragma unroll
        for (int v = 0; v < V8; v++) {
            const float4 qa = *(const float4*)(qh + (v * 8 + l8) * 8);
            const float4 qb = *(const float4*)(qh + (v * 8 + l8) * 8 + 4);
            q[h][v * 8 + 0] = qa.x * a.scale; q[h][v * 8 + 1] = qa.y * a.scale;
            q[h][v * 8 + 2] = qa.z * a.scale; q[h][v * 8 + 3] = qa.w * a.scale;
            q[h][v * 8 + 4] = qb.x * a.scale; q[h][v * 8 + 5] = qb.y * a.scale;
            q[h][v * 8 + 6] = qb.z * a.scale; q[h][v * 8 + 7] = qb.w * a.scale;
        }
    }
    // ---- scores ---------------------------------------------------------------------------------
    float sc[NIT][GQ], mx[GQ];
#pragma unroll
    for (int h = 0; h < GQ; h++) mx[h] = -INFINITY;
#pragma unroll
    for (int i = 0; i < NIT; i++) {
        float dot[GQ];
#pragma unroll
        for (int h = 0; h < GQ; h++) dot[h] = 0.f;
#pragma unroll
        for (int v = 0; v < V8; v++) {
            const uint32_t kw[4] = {kreg[i][v].x, kreg[i][v].y, kreg[i][v].z, kreg[i][v].w};
#pragma unroll
            for (int e = 0; e < 4; e++) {
                const float k0 = __uint_as_float(kw[e] << 16), k1 = __uint_as_float(kw[e] & 0xffff0000u);
#pragma unroll
                for (int h = 0; h < GQ; h++) dot[h] = fmaf(q[h][v * 8 + 2 * e + 1], k1, fmaf(q[h][v * 8 + 2 * e], k0, dot[h]));
            }
        }
#pragma unroll
        for (int h = 0; h < GQ; h++) {
            float d = dot[h];
            d += __shfl_xor_sync(0xffffffffu, d, 1);
            d += __shfl_xor_sync(0xffffffffu, d, 2);
            d += __shfl_xor_sync(0xffffffffu, d, 4);
            sc[i][h] = valid[i] ? d : -INFINITY;
            mx[h] = fmaxf(mx[h], sc[i][h]);
        }
    }
#pragma unroll
    for (int h = 0; h < GQ; h++) {
        const float m = warp_max(mx[h]);
        if (lane == 0) smax[h][warp] = m;
    }
    __syncthreads();
    float cmax[GQ];
#pragma unroll
    for (int h = 0; h < GQ; h++) cmax[h] = fmaxf(fmaxf(smax[h][0], smax[h][1]), fmaxf(smax[h][2], smax[h][3]));
    // ---- weights and weighted values ---------------------------------------------------------------
    float acc[GQ][E], lsum[GQ];
#pragma unroll
    for (int h = 0; h < GQ; h++) {
        lsum[h] = 0.f;
#pragma unroll
        for (int e = 0; e < E; e++) acc[h][e] = 0.f;
    }
#pragma unroll
    for (int i = 0; i < NIT; i++) {
        float w[GQ];
#pragma unroll
        for (int h = 0; h < GQ; h++) { w[h] = valid[i] ? __expf(sc[i][h] - cmax[h]) : 0.f; lsum[h] += w[h]; }
#pragma unroll
        for (int v = 0; v < V8; v++) {
            const uint32_t vw[4] = {vreg[i][v].x, vreg[i][v].y, vreg[i][v].z, vreg[i][v].w};
#pragma unroll
            for (int e = 0; e < 4; e++) {
                const float v0 = __uint_as_float(vw[e] << 16), v1 = __uint_as_float(vw[e] & 0xffff0000u);
#pragma unroll
                for (int h = 0; h < GQ; h++) {
                    acc[h][v * 8 + 2 * e] = fmaf(w[h], v0, acc[h][v * 8 + 2 * e]);
                    acc[h][v * 8 + 2 * e + 1] = fmaf(w[h], v1, acc[h][v * 8 + 2 * e + 1]);
                }
            }
        }
    }
    // combine the 4 position groups of a warp, then the 4 warps
#pragma unroll
    for (int h = 0; h < GQ; h++) {
#pragma unroll
        for (int e = 0; e < E; e++) {
            float v = acc[h][e];
            v += __shfl_xor_sync(0xffffffffu, v, 8);
            v += __shfl_xor_sync(0xffffffffu, v, 16);
            acc[h][e] = v;
        }
        float l = (l8 == 0) ? lsum[h] : 0.f;  // the 8 lanes of a group hold the same weight: count it once
        l = warp_sum(l);
        if (lane == 0) ssum[h][warp] = l;
        if (lane < 8) {
#pragma unroll
            for (int v = 0; v < V8; v++)
#pragma unroll
                for (int e = 0; e < 8; e++) red[warp][h][(v * 8 + l8) * 8 + e] = acc[h][v * 8 + e];
        }
    }
    __syncthreads();
    for (int idx = tid; idx < GQ * D; idx += 128) {
        const int h = idx / D, d = idx - h * D;
        const float v = red[0][h][d] + red[1][h][d] + red[2][h][d] + red[3][h][d];
        const float l = ssum[h][0] + ssum[h][1] + ssum[h][2] + ssum[h][3];
        const int qh = qh0 + h;
        if (a.nchunks == 1) {
            a.out[((int64_t)row * a.Hq + qh) * D + d] = v / l;
        } else {
            float* pa = a.part + (((int64_t)row * a.Hq + qh) * a.nchunks + chunk) * (D + 2);
            pa[d] = v;
            if (d == 0) { pa[D] = cmax[h]; pa[D + 1] = l; }
        }
    }
}

template <int D, int GQ>
__global__ void __launch_bounds__(128) sdpa_decode_tiles_kernel(const SdpaArgs a) {
    pdl_trigger();
    pdl_wait();
    constexpr int E = D / 8;          // elements per lane
    constexpr int V8 = E / 8;         // 16-byte loads per lane per row
    constexpr int NIT = 512 / D > 0 ? 512 / D : 1;  // positions per lane group and tile: a tile is 16*NIT positions
    constexpr int TILE = 16 * NIT;
    __shared__ float red[4][GQ][D + 2];
    __shared__ float smax[GQ][4], ssum[GQ][4];

    // blockIdx.x indexes a bundle of GQ consecutive query heads that share one kv head
    const int row = blockIdx.z, chunk = blockIdx.y;
    const int qh0 = blockIdx.x * GQ, kvh = qh0 / (a.Hq / a.Hkv);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int l8 = lane & 7, pg = warp * 4 + (lane >> 3);  // position group 0..15
    const int ctx = a.row_pos[row] + 1;                    // keys 0..pos inclusive
    const int lo = a.window > 0 ? max(0, ctx - a.window) : 0;  // sliding block: keys lo..pos
    const int c0 = chunk * a.chunk_len;                    // a chunk is one or more tiles, walked with a running softmax
    if (c0 >= ctx || c0 + a.chunk_len <= lo) return;
    const int c1 = min(c0 + a.chunk_len, ctx);
    const int KR = a.Hkv * D;
    const uint16_t* kbase = a.kcache + (int64_t)a.row_lane[row] * a.lane_stride + (int64_t)kvh * D;
    const uint16_t* vbase = a.vcache + (int64_t)a.row_lane[row] * a.lane_stride + (int64_t)kvh * D;

    float q[GQ][E];  // query slices of this lane for the GQ heads (filled behind the first tile's loads)
    // running state of this warp over its positions: maximum, sum of weights, weighted values
    float mrun[GQ], lsum[GQ], acc[GQ][E];
#pragma unroll
    for (int h = 0; h < GQ; h++) {
        mrun[h] = -INFINITY; lsum[h] = 0.f;
#pragma unroll
        for (int e = 0; e < E; e++) acc[h][e] = 0.f;
    }
    const int t0 = c0 + (lo > c0 ? (lo - c0) / TILE * TILE : 0);  // tiles wholly below the window are skipped
    for (int p0 = t0; p0 < c1; p0 += TILE) {
        // ---- every load of the tile goes out first --------------------------------------------
        uint4 kreg[NIT][V8], vreg[NIT][V8];
        bool valid[NIT];
#pragma unroll
        for (int i = 0; i < NIT; i++) {
            const int p = p0 + pg + 16 * i;
            valid[i] = p < ctx && p >= lo;
            const int64_t off = (int64_t)(valid[i] ? p : min(max(p0, lo), ctx - 1)) * KR;
#pragma unroll
            for (int v = 0; v < V8; v++) {
                kreg[i][v] = __ldg((const uint4*)(kbase + off + (v * 8 + l8) * 8));
                vreg[i][v] = __ldg((const uint4*)(vbase + off + (v * 8 + l8) * 8));
            }
        }
        if (p0 == t0) {
            // the query, pre-multiplied by the softmax scale: loaded while the first tile's keys and values are in flight
#pragma unroll
            for (int h = 0; h < GQ; h++) {
                const float* qh = a.q + ((int64_t)row * a.Hq + qh0 + h) * D;
#pragma unroll
                for (int v = 0; v < V8; v++) {
                    const float4 qa = *(const float4*)(qh + (v * 8 + l8) * 8);
                    const float4 qb = *(const float4*)(qh + (v * 8 + l8) * 8 + 4);
                    q[h][v * 8 + 0] = qa.x * a.scale; q[h][v * 8 + 1] = qa.y * a.scale;
                    q[h][v * 8 + 2] = qa.z * a.scale; q[h][v * 8 + 3] = qa.w * a.scale;
                    q[h][v * 8 + 4] = qb.x * a.scale; q[h][v * 8 + 5] = qb.y * a.scale;
                    q[h][v * 8 + 6] = qb.z * a.scale; q[h][v * 8 + 7] = qb.w * a.scale;
                }
            }
        }
        // ---- scores ---------------------------------------------------------------------------
        float sc[NIT][GQ], mx[GQ];
#pragma unroll
        for (int h = 0; h < GQ; h++) mx[h] = -INFINITY;
#pragma unroll
        for (int i = 0; i < NIT; i++) {
            float dot[GQ];
#pragma unroll
            for (int h = 0; h < GQ; h++) dot[h] = 0.f;
#pragma unroll
            for (int v = 0; v < V8; v++) {
                const uint32_t kw[4] = {kreg[i][v].x, kreg[i][v].y, kreg[i][v].z, kreg[i][v].w};
#pragma unroll
                for (int e = 0; e < 4; e++) {
                    const float k0 = __uint_as_float(kw[e] << 16), k1 = __uint_as_float(kw[e] & 0xffff0000u);
#pragma unroll
                    for (int h = 0; h < GQ; h++) dot[h] = fmaf(q[h][v * 8 + 2 * e + 1], k1, fmaf(q[h][v * 8 + 2 * e], k0, dot[h]));
                }
            }
#pragma unroll
            for (int h = 0; h < GQ; h++) {
                float d = dot[h];
                d += __shfl_xor_sync(0xffffffffu, d, 1);
                d += __shfl_xor_sync(0xffffffffu, d, 2);
                d += __shfl_xor_sync(0xffffffffu, d, 4);
                sc[i][h] = valid[i] ? d : -INFINITY;
                mx[h] = fmaxf(mx[h], sc[i][h]);
            }
        }
        // ---- running softmax of the warp: rescale what it has, add the tile -----------------------
        float mref[GQ];
#pragma unroll
        for (int h = 0; h < GQ; h++) {
            const float mnew = fmaxf(mrun[h], warp_max(mx[h]));
            mref[h] = mnew == -INFINITY ? 0.f : mnew;      // no visible key yet: keep exp() finite
            const float rescale = __expf(mrun[h] - mref[h]);  // -inf -> 0
            mrun[h] = mnew;
            lsum[h] *= rescale;
#pragma unroll
            for (int e = 0; e < E; e++) acc[h][e] *= rescale;
        }
#pragma unroll
        for (int i = 0; i < NIT; i++) {
            float w[GQ];
#pragma unroll
            for (int h = 0; h < GQ; h++) { w[h] = valid[i] ? __expf(sc[i][h] - mref[h]) : 0.f; lsum[h] += w[h]; }
#pragma unroll
            for (int v = 0; v < V8; v++) {
                const uint32_t vw[4] = {vreg[i][v].x, vreg[i][v].y, vreg[i][v].z, vreg[i][v].w};
#pragma unroll
                for (int e = 0; e < 4; e++) {
                    const float v0 = __uint_as_float(vw[e] << 16), v1 = __uint_as_float(vw[e] & 0xffff0000u);
#pragma unroll
                    for (int h = 0; h < GQ; h++) {
                        acc[h][v * 8 + 2 * e] = fmaf(w[h], v0, acc[h][v * 8 + 2 * e]);
                        acc[h][v * 8 + 2 * e + 1] = fmaf(w[h], v1, acc[h][v * 8 + 2 * e + 1]);
                    }
                }
            }
        }
    }
    // combine the 4 position groups of a warp, then the 4 warps (each with its own maximum)
#pragma unroll
    for (int h = 0; h < GQ; h++) {
#pragma unroll
        for (int e = 0; e < E; e++) {
            float v = acc[h][e];
            v += __shfl_xor_sync(0xffffffffu, v, 8);
            v += __shfl_xor_sync(0xffffffffu, v, 16);
            acc[h][e] = v;
        }
        float l = (l8 == 0) ? lsum[h] : 0.f;  // the 8 lanes of a group hold the same weight: count it once
        l = warp_sum(l);
        if (lane == 0) { ssum[h][warp] = l; smax[h][warp] = mrun[h]; }
        if (lane < 8) {
#pragma unroll
            for (int v = 0; v < V8; v++)
#pragma unroll
                for (int e = 0; e < 8; e++) red[warp][h][(v * 8 + l8) * 8 + e] = acc[h][v * 8 + e];
        }
    }
    __syncthreads();
    for (int idx = tid; idx < GQ * D; idx += 128) {
        const int h = idx / D, d = idx - h * D;
        const float m = fmaxf(fmaxf(smax[h][0], smax[h][1]), fmaxf(smax[h][2], smax[h][3]));  // finite: the chunk holds a visible key
        float v = 0.f, l = 0.f;
#pragma unroll
        for (int w = 0; w < 4; w++) {
            const float e = __expf(smax[h][w] - m);  // a warp without a visible key: exp(-inf) = 0
            v = fmaf(red[w][h][d], e, v);
            l = fmaf(ssum[h][w], e, l);
        }
        const int qh = qh0 + h;
        if (a.nchunks == 1) {
            a.out[((int64_t)row * a.Hq + qh) * D + d] = v / l;
        } else {
            float* pa = a.part + (((int64_t)row * a.Hq + qh) * a.nchunks + chunk) * (D + 2);
            pa[d] = v;
            if (d == 0) { pa[D] = m; pa[D + 1] = l; }
        }
    }
}

// stage 2: merge chunk partials with their log-sum-exp weights. One CTA per (head, row), four
// warps; warp w takes chunks w, w+4, ... and each lane D/32 consecutive dimensions. A single pass:
// a warp issues the loads of (max, sum, accumulator slice) of up to MERGE_BATCH of its chunks
// together, folds them into a running (max, sum, accumulator) of its own, and the four warps' states
// meet once in shared memory - one memory round trip per MERGE_BATCH*4 chunks instead of the three
// dependent passes (maxima, weights, accumulators) of a two-level softmax merge.
constexpr int MERGE_BATCH = 8;
template <int D>
__global__ void __launch_bounds__(128) sdpa_merge_kernel(const float* __restrict__ part,
                                                         const int32_t* __restrict__ row_pos, int Hq, int nchunks,
                                                         int chunk_len, float* __restrict__ out,
                                                         uint16_t* __restrict__ cols, int split, int window) {
    pdl_trigger();
    pdl_wait();
    constexpr int DL = D / 32;  // dimensions per lane (2, 4, 8 or 16)
    __shared__ float sm_m[4], sm_l[4];
    __shared__ float acc_s[4][D];
    const int row = blockIdx.y, qh = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int ctx = row_pos[row] + 1;
    const int used = min(nchunks, (ctx + chunk_len - 1) / chunk_len);
    const int first = window > 0 ? max(0, ctx - window) / chunk_len : 0;  // chunks below the window wrote nothing
    const float* pa = part + ((int64_t)row * Hq + qh) * nchunks * (D + 2);
    float m = -INFINITY, l = 0.f, acc[DL];
#pragma unroll
    for (int i = 0; i < DL; i++) acc[i] = 0.f;
    for (int c0 = first + warp; c0 < used; c0 += 4 * MERGE_BATCH) {
        float cm[MERGE_BATCH], cl[MERGE_BATCH];
        float2 cv[MERGE_BATCH][DL / 2];
#pragma unroll
        for (int b = 0; b < MERGE_BATCH; b++) {
            const int c = c0 + 4 * b;
            const bool live = c < used;
            const float* p = pa + (int64_t)(live ? c : c0) * (D + 2);
            cm[b] = live ? p[D] : -INFINITY;
            cl[b] = live ? p[D + 1] : 0.f;
            const float2* src = (const float2*)(p + lane * DL);  // rows are 8-byte aligned
#pragma unroll
            for (int i = 0; i < DL / 2; i++) cv[b][i] = src[i];
        }
        float bm = m;
#pragma unroll
        for (int b = 0; b < MERGE_BATCH; b++) bm = fmaxf(bm, cm[b]);
        if (bm == -INFINITY) continue;
        const float rescale = __expf(m - bm);  // m = -inf -> 0
        l *= rescale;
#pragma unroll
        for (int i = 0; i < DL; i++) acc[i] *= rescale;
#pragma unroll
        for (int b = 0; b < MERGE_BATCH; b++) {
            const float w = __expf(cm[b] - bm);  // dead slots: exp(-inf) = 0
            l = fmaf(cl[b], w, l);
#pragma unroll
            for (int i = 0; i < DL / 2; i++) {
                acc[2 * i] = fmaf(cv[b][i].x, w, acc[2 * i]);
                acc[2 * i + 1] = fmaf(cv[b][i].y, w, acc[2 * i + 1]);
            }
        }
        m = bm;
    }
    if (lane == 0) { sm_m[warp] = m; sm_l[warp] = l; }
#pragma unroll
    for (int i = 0; i < DL; i++) acc_s[warp][lane * DL + i] = acc[i];
    __syncthreads();
    const float gm = fmaxf(fmaxf(sm_m[0], sm_m[1]), fmaxf(sm_m[2], sm_m[3]));
    float w4[4], denom = 0.f;
#pragma unroll
    for (int w = 0; w < 4; w++) { w4[w] = __expf(sm_m[w] - gm); denom = fmaf(sm_l[w], w4[w], denom); }
    for (int d = tid; d < D; d += 128) {
        const float o = (acc_s[0][d] * w4[0] + acc_s[1][d] * w4[1] + acc_s[2][d] * w4[2] + acc_s[3][d] * w4[3]) / denom;
        out[((int64_t)row * Hq + qh) * D + d] = o;
        if (cols) store_split(cols, split, row, Hq * D, qh * D + d, o);
    }
}

// ---- decode attention in one kernel ---------------------------------------------------------
// Per-head RMSNorm + RoPE of q and of the new key, the KV append, split-KV attention and the merge
// of the chunk partials (by the last CTA of a kv head to finish, through a counter) in one launch
// instead of three (qknorm_rope_append, sdpa_decode, sdpa_merge): grid (kv head, key chunk, row).
// The item itself is attn_item.cuh, shared with the one-kernel decode step.
template <int D, int GQ>
__global__ void __launch_bounds__(128) sdpa_fused_kernel(const SdpaFusedArgs a) {
    pdl_trigger();
    pdl_wait();
    __shared__ AttnItemSmem<D, GQ> s;
    constexpr int CH = 16 * (512 / D > 0 ? 512 / D : 1);
    const int kvh = blockIdx.x, chunk = blockIdx.y, row = blockIdx.z;
    const int pos = a.row_pos[row];
    const int used = min(a.nchunks, (pos + CH) / CH);
    if (chunk >= used) return;
    AttnItemArgs it;
    it.qkv = a.qkv + (int64_t)row * (a.Hq + 2 * a.Hkv) * D;
    it.n_q = a.n_q; it.n_k = a.n_k; it.rope = a.rope;
    const int64_t lane_off = (int64_t)a.row_lane[row] * a.lane_stride;
    it.kc = a.kcache + lane_off; it.vc = a.vcache + lane_off;
    it.part = a.part + (int64_t)row * a.Hq * a.nchunks * (D + 2);
    it.counter = a.counters + (int64_t)row * a.Hkv;
    it.Hq = a.Hq; it.Hkv = a.Hkv; it.nchunks_cap = a.nchunks; it.max_len = a.max_len;
    it.eps = a.eps; it.scale = a.scale;
    attn_item<D, GQ>(it, s, [] { __syncthreads(); },
                     [&](AttnItemSmem<D, GQ>& sm, int qh0) {
                         for (int idx = threadIdx.x; idx < GQ * D; idx += 128) {
                             const int h = idx / D, d = idx - h * D;
                             const float v = sm.q[h][d];
                             a.out[((int64_t)row * a.Hq + qh0 + h) * D + d] = v;
                             if (a.cols) store_split(a.cols, a.split, row, a.Hq * D, (qh0 + h) * D + d, v);
                         }
                     },
                     kvh, chunk, used, pos);
}

bool sdpa_fused_supported(int Hq, int Hkv, int D) { return Hq == 2 * Hkv && (D == 64 || D == 128 || D == 256); }

int32_t launch_sdpa_fused(cudaStream_t s, const SdpaFusedArgs& a, int rows, int D) {
    if (!sdpa_fused_supported(a.Hq, a.Hkv, D)) return fail(LTHN_ERR_INVALID, "sdpa_fused: needs two query heads per kv head and head_dim 64, 128 or 256");
    dim3 grid(a.Hkv, a.nchunks, rows);
    if (D == 64) LTHN_CUDA_TRY(launch_k(sdpa_fused_kernel<64, 2>, grid, dim3(128), 0, s, a));
    else if (D == 128) LTHN_CUDA_TRY(launch_k(sdpa_fused_kernel<128, 2>, grid, dim3(128), 0, s, a));
    else LTHN_CUDA_TRY(launch_k(sdpa_fused_kernel<256, 2>, grid, dim3(128), 0, s, a));
    return LTHN_OK;
}

// ---- greedy argmax --------------------------------------------------------------------
// Strict '>' with the lowest index winning ties (model.Greedy, model/sample.go:33-50;
// hipReferenceGreedySample). Two stages: per-block best, then one block per row.
__device__ __forceinline__ void argmax_merge(float& v, int& i, float ov, int oi) {
    if (ov > v || (ov == v && oi < i)) { v = ov; i = oi; }
}
__global__ void argmax_stage1_kernel(const float* __restrict__ logits, int V, int blocks_per_row,
                                     float* __restrict__ pv, int* __restrict__ pi) {
    pdl_trigger();
    pdl_wait();
    __shared__ float sv[32];
    __shared__ int si[32];
    const int row = blockIdx.y;
    const float* lr = logits + (int64_t)row * V;
    float v = -INFINITY;
    int idx = 0x7fffffff;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < V; i += gridDim.x * blockDim.x) argmax_merge(v, idx, lr[i], i);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) argmax_merge(v, idx, __shfl_xor_sync(0xffffffffu, v, o), __shfl_xor_sync(0xffffffffu, idx, o));
    if ((threadIdx.x & 31) == 0) { sv[threadIdx.x >> 5] = v; si[threadIdx.x >> 5] = idx; }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < (blockDim.x >> 5); w++) argmax_merge(v, idx, sv[w], si[w]);
        pv[row * blocks_per_row + blockIdx.x] = v;
        pi[row * blocks_per_row + blockIdx.x] = idx;
    }
}
__global__ void argmax_stage2_kernel(const float* __restrict__ pv, const int* __restrict__ pi, int blocks_per_row,
                                     int32_t* __restrict__ out_idx, float* __restrict__ out_val, int index_offset) {
    pdl_trigger();
    pdl_wait();
    const int row = blockIdx.x;
    float v = -INFINITY;
    int idx = 0x7fffffff;
    for (int i = threadIdx.x; i < blocks_per_row; i += 32) argmax_merge(v, idx, pv[row * blocks_per_row + i], pi[row * blocks_per_row + i]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) argmax_merge(v, idx, __shfl_xor_sync(0xffffffffu, v, o), __shfl_xor_sync(0xffffffffu, idx, o));
    if (threadIdx.x == 0) {
        out_idx[row] = idx + index_offset;
        if (out_val) out_val[row] = v;
    }
}

// advance per-row positions and feed the chosen token back (one decode step bookkeeping)
__global__ void advance_kernel(int32_t* row_pos, int32_t* ids, const int32_t* next, int rows) {
    const int r = blockIdx.x * blockDim.x + threadIdx.x;
    if (r < rows) { row_pos[r] += 1; ids[r] = next[r]; }
}

// act = gelu_tanh(gate) * up for a block whose gate and up projections ran as separate matvecs
// (8-bit codes); gelu_tanh as hipGemma4Q4HostGELU (engine/hip/hip_gemma4_q4_layer.go:3582-3597)
__global__ void geglu_kernel(const float* __restrict__ g, const float* __restrict__ u, float* __restrict__ out, int64_t n) {
    pdl_trigger();
    pdl_wait();
    const float k0 = 0.7978845608028654f, k1 = 0.044715f;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
        const float x = g[i];
        const float inner = k0 * (x + k1 * x * x * x);
        out[i] = 0.5f * x * (1.0f + tanhf(inner)) * u[i];
    }
}

// ---- launch wrappers ----------------------------------------------------------------------
int32_t launch_geglu(cudaStream_t s, const float* g, const float* u, float* out, int64_t n) {
    const unsigned grid = (unsigned)std::min<int64_t>((n + 255) / 256, 148 * 8);
    LTHN_CUDA_TRY(launch_k(geglu_kernel, dim3(grid), dim3(256), 0, s, g, u, out, n));
    return LTHN_OK;
}

int32_t launch_embed(cudaStream_t s, const int32_t* ids, int rows, const uint32_t* packed, const uint16_t* scales,
                     const uint16_t* biases, int hidden, int vocab, float embed_scale, float* out) {
    LTHN_CUDA_TRY(launch_k(embed_kernel, dim3(rows), dim3(256), 0, s, ids, packed, scales, biases, hidden, vocab, embed_scale, out));
    return LTHN_OK;
}

int32_t launch_rmsnorm(cudaStream_t s, const float* a, float* h, const float* w_post, const float* w_next, float* out,
                       int rows, int width, float eps, int mode, uint16_t* cols, int split) {
    // one CTA per row; enough threads that each handles two or three elements (the f64 sum of
    // squares and the IEEE divisions are latency, not throughput, so parallelism is what helps)
    const int threads = width >= 2048 ? 1024 : (width >= 512 ? 512 : 256);
    const bool aligned = (((uintptr_t)a | (uintptr_t)h | (uintptr_t)w_post | (uintptr_t)w_next | (uintptr_t)out) & 15) == 0;
    if (rows > 64 && width % 4 == 0 && aligned)  // many rows (prefill): a warp per row
        LTHN_CUDA_TRY(launch_k(rmsnorm_rows_kernel, dim3((rows + 3) / 4), dim3(128), 0, s, a, h, w_post, w_next, out, rows, width, eps, mode, cols, split));
    else if (width <= 8 * threads)
        LTHN_CUDA_TRY(launch_k(rmsnorm_reg_kernel, dim3(rows), dim3(threads), 0, s, a, h, w_post, w_next, out, width, eps, mode, cols, split));
    else
        LTHN_CUDA_TRY(launch_k(rmsnorm_kernel, dim3(rows), dim3(threads), 0, s, a, h, w_post, w_next, out, width, eps, mode, cols, split));
    return LTHN_OK;
}

int32_t launch_rmsnorm_gather(cudaStream_t s, const PeerGather& pg, float* h, const float* w_post, const float* w_next,
                              float* out, int rows, int width, float eps, uint16_t* cols, int split) {
    if (width > 8192) return fail(LTHN_ERR_INVALID, "rmsnorm_gather: width above 8192");
    if (pg.t < 2 || pg.t > 8) return fail(LTHN_ERR_INVALID, "rmsnorm_gather: 2 to 8 ranks");
    const int threads = width >= 2048 ? 1024 : (width >= 512 ? 512 : 256);
    LTHN_CUDA_TRY(launch_k(rmsnorm_gather_kernel, dim3(rows), dim3(threads), 0, s, pg, h, w_post, w_next, out, width, eps, cols, split));
    return LTHN_OK;
}

int32_t launch_qknorm_rope_append(cudaStream_t s, const float* qkv, const float* q_norm, const float* k_norm,
                                  const float2* rope_table, const int32_t* row_pos, const int32_t* row_lane,
                                  float* q_out, uint16_t* kcache, uint16_t* vcache, int rows, int Hq, int Hkv, int D,
                                  float eps, int64_t lane_stride, int max_len) {
    dim3 grid(rows, Hq + 2 * Hkv);
    LTHN_CUDA_TRY(launch_k(qknorm_rope_append_kernel, grid, dim3(D / 2), 0, s, qkv, q_norm, k_norm, rope_table, row_pos, row_lane,
                           q_out, kcache, vcache, Hq, Hkv, D, eps, lane_stride, max_len, 1.0 / (double)D));
    return LTHN_OK;
}

int32_t launch_rmsnorm_rope(cudaStream_t s, const float* x, const float* w, const int32_t* positions, float* out,
                            int rows, int heads, int D, int rotary, float eps, float rope_base, int bf16_seams) {
    dim3 grid(rows, heads);
    rmsnorm_rope_kernel<<<grid, D / 2, 0, s>>>(x, w, positions, out, heads, D, rotary, eps, rope_base, bf16_seams);
    LTHN_CUDA_TRY(cudaGetLastError());
    return LTHN_OK;
}

int sdpa_chunking(int max_ctx, int D, int* chunk_len, int rows, int bundles) {
    // A tile is what a CTA holds in registers with all its loads in flight (8192/D keys); a chunk is one or
    // more tiles walked with a running softmax. One tile per chunk while that keeps the grid under ~2.5 CTAs
    // per SM (few heads: the 26-layer model decodes 6 % slower with two tiles per chunk) and whenever more
    // than two rows share the launch (16 lanes: 5 % slower with long chunks - the grid is full anyway and a
    // CTA's tiles are a serial chain); beyond that, longer chunks mean fewer partials for the merge and fewer
    // CTA prologues (62-layer model, one row, 4096 keys: 3 tiles per chunk, 2-3.5 % faster per token).
    // LTHN_CUDA_SDPA_TILES=n forces n tiles per chunk.
    const int nit = 512 / D > 0 ? 512 / D : 1, tile = 16 * nit;
    const int tiles = (max_ctx + tile - 1) / tile;
    static const int forced = [] { const char* e = getenv("LTHN_CUDA_SDPA_TILES"); return e ? atoi(e) : 0; }();
    int tl = rows <= 2 ? (int)((int64_t)tiles * std::max(1, rows * bundles) / 370) : 1;
    tl = std::min(4, tl);
    if (forced > 0) tl = forced;
    tl = std::min(8, std::max(1, tl));
    *chunk_len = tile * tl;
    return (max_ctx + *chunk_len - 1) / *chunk_len;
}

// chunks of one tile each: what the one-launch attention and the one-kernel decode step use
int sdpa_item_chunks(int max_ctx, int D) {
    const int nit = 512 / D > 0 ? 512 / D : 1, tile = 16 * nit;
    return (max_ctx + tile - 1) / tile;
}

size_t sdpa_scratch_bytes(int rows, int Hq, int D, int nchunks) {
    return (size_t)rows * Hq * nchunks * (D + 2) * sizeof(float);
}

// bundle = query heads handled per CTA (they share K/V loads); must divide the GQA group
template <int D>
static int32_t launch_sdpa_d(cudaStream_t s, const SdpaArgs& a, int rows, int bundle) {
    dim3 grid(a.Hq / bundle, a.nchunks, rows);
    constexpr int TILE = 16 * (512 / D > 0 ? 512 / D : 1);
    if (rows <= 2 || a.chunk_len > TILE) {  // one or two rows (latency matters, the grid is small) or several tiles per chunk
        switch (bundle) {
            case 1: LTHN_CUDA_TRY(launch_k(sdpa_decode_tiles_kernel<D, 1>, grid, dim3(128), 0, s, a)); break;
            case 2: if (D <= 256) { LTHN_CUDA_TRY(launch_k(sdpa_decode_tiles_kernel<(D <= 256 ? D : 64), 2>, grid, dim3(128), 0, s, a)); break; }
            case 4: if (D <= 128) { LTHN_CUDA_TRY(launch_k(sdpa_decode_tiles_kernel<(D <= 128 ? D : 64), 4>, grid, dim3(128), 0, s, a)); break; }
            default: return fail(LTHN_ERR_INVALID, "sdpa_decode: unsupported head bundle");
        }
        return LTHN_OK;
    }
    switch (bundle) {
        case 1: LTHN_CUDA_TRY(launch_k(sdpa_decode_kernel<D, 1>, grid, dim3(128), 0, s, a)); break;
        case 2: if (D <= 256) { LTHN_CUDA_TRY(launch_k(sdpa_decode_kernel<(D <= 256 ? D : 64), 2>, grid, dim3(128), 0, s, a)); break; }
        case 4: if (D <= 128) { LTHN_CUDA_TRY(launch_k(sdpa_decode_kernel<(D <= 128 ? D : 64), 4>, grid, dim3(128), 0, s, a)); break; }
        default: return fail(LTHN_ERR_INVALID, "sdpa_decode: unsupported head bundle");
    }
    return LTHN_OK;
}

int32_t launch_sdpa_decode(cudaStream_t s, SdpaArgs a, int rows, int D) {
    if (a.Hq % a.Hkv != 0) return fail(LTHN_ERR_INVALID, "sdpa_decode: Hq must be a multiple of Hkv");
    const int GQ = a.Hq / a.Hkv;
    if (a.nchunks > 1 && !a.part) return fail(LTHN_ERR_INVALID, "sdpa_decode: split-KV needs a scratch buffer");
    // register budget: bundle * D/8 accumulators and as many query values per lane
    const int max_bundle = D <= 128 ? 4 : (D <= 256 ? 2 : 1);
    int bundle = 1;
    for (int c = max_bundle; c >= 1; c >>= 1)
        if (GQ % c == 0) { bundle = c; break; }
    int32_t rc;
    if (D == 128) rc = launch_sdpa_d<128>(s, a, rows, bundle);
    else if (D == 256) rc = launch_sdpa_d<256>(s, a, rows, bundle);
    else if (D == 64) rc = launch_sdpa_d<64>(s, a, rows, bundle);
    else if (D == 512) rc = launch_sdpa_d<512>(s, a, rows, bundle);
    else return fail(LTHN_ERR_INVALID, "sdpa_decode: head_dim must be 64, 128, 256 or 512");
    if (rc) return rc;
    if (a.nchunks > 1) {
        dim3 grid(a.Hq, rows);
        const float* cpart = a.part;
        if (D == 64) LTHN_CUDA_TRY(launch_k(sdpa_merge_kernel<64>, grid, dim3(128), 0, s, cpart, a.row_pos, a.Hq, a.nchunks, a.chunk_len, a.out, a.cols, a.split, a.window));
        else if (D == 128) LTHN_CUDA_TRY(launch_k(sdpa_merge_kernel<128>, grid, dim3(128), 0, s, cpart, a.row_pos, a.Hq, a.nchunks, a.chunk_len, a.out, a.cols, a.split, a.window));
        else if (D == 256) LTHN_CUDA_TRY(launch_k(sdpa_merge_kernel<256>, grid, dim3(128), 0, s, cpart, a.row_pos, a.Hq, a.nchunks, a.chunk_len, a.out, a.cols, a.split, a.window));
        else LTHN_CUDA_TRY(launch_k(sdpa_merge_kernel<512>, grid, dim3(128), 0, s, cpart, a.row_pos, a.Hq, a.nchunks, a.chunk_len, a.out, a.cols, a.split, a.window));
    }
    return LTHN_OK;
}

int32_t launch_argmax(cudaStream_t s, const float* logits, int rows, int V, float* pv, int* pi, int32_t* out_idx,
                      float* out_val, int index_offset) {
    const int bpr = ARGMAX_BLOCKS;
    dim3 grid(bpr, rows);
    LTHN_CUDA_TRY(launch_k(argmax_stage1_kernel, grid, dim3(256), 0, s, logits, V, bpr, pv, pi));
    LTHN_CUDA_TRY(launch_k(argmax_stage2_kernel, dim3(rows), dim3(32), 0, s, (const float*)pv, (const int*)pi, bpr, out_idx, out_val, index_offset));
    return LTHN_OK;
}

int32_t launch_advance(cudaStream_t s, int32_t* row_pos, int32_t* ids, const int32_t* next, int rows) {
    advance_kernel<<<(rows + 63) / 64, 64, 0, s>>>(row_pos, ids, next, rows);
    LTHN_CUDA_TRY(cudaGetLastError());
    return LTHN_OK;
}

}  // namespace lthn
