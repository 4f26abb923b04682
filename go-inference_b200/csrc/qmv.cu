// qmv.cu — affine_qmv: decode-time MLX-affine 4-bit matvec for 1..32 activation
// rows, written for B200 (sm_100a).
//
// y[m,n] = sum_k x[m,k] * (scale[n,k/64] * code[n,k] + bias[n,k/64])
//
// The kernel is a pure weight stream (0.5625 B per weight element: 4-bit code +
// one bf16 scale and bias per 64) and is bound by HBM bandwidth, so the design
// goal is to spend as few issue slots per byte as possible:
//
//  * Each warp owns whole quantisation groups (64 consecutive k) of a 16-row
//    tile. A lane loads 8 bytes (16 codes) of row r and of row r+8; the four
//    lanes of a quad cover one 32-byte group segment of a row, so a warp-wide
//    load touches eight full 32-byte sectors.
//  * Codes are expanded to bf16 with one logic op each: (w>>4i & 0x000F000F) |
//    0x43004300 is the bf16 pair {128+q_lo, 128+q_hi}. The dot products run on
//    the tensor cores (mma.sync m16n8k16, bf16 x bf16 -> f32): weights are the
//    16-row A operand, up to 8 activation columns are the B operand, so one
//    weight pass serves 8 activation columns for the price of one.
//    The k order inside an MMA is permuted identically for A and B, which a dot
//    product does not care about; that is what lets the code pairs come out of
//    the packed word without any shuffling.
//  * Per group the f32 accumulator D_g = sum (128+q) x is folded as
//    acc += scale*D_g + (bias - 128*scale)*X_g with X_g = sum x, which a second MMA
//    against an all-ones A operand yields in exactly the lanes that need it (the fused
//    GeGLU form, whose MMA count is highest, forms X_g with f32 adds and shuffles instead).
//  * f32 activations are supplied as 2 or 3 bf16 columns (hi/mid/lo split, exact
//    to 16/24 mantissa bits) whose results are added in the epilogue, so the
//    tensor-core path keeps f32-grade activations.
//  * The bf16 scale/bias tile of the CTA's rows is staged into shared memory by
//    one 1-D bulk (TMA) copy per tensor; warps split K and are summed in a fixed
//    order through shared memory (deterministic, no atomics).
//
// A second, general kernel (one warp per row, SIMT) serves the other widths of
// the format (2/8 bit, group 32/128) that the reference's fixtures exercise.
#include "common.cuh"
#include "qmv.hpp"

#include <algorithm>
#include <mutex>

namespace lthn {

struct QmvArgs {
    const uint32_t* wq;      // [N, K/8]
    const uint16_t* scales;  // [N, K/64]
    const uint16_t* biases;  // [N, K/64]
    const uint16_t* x;       // [C, K] bf16 activation columns
    void* y;                 // [M, N]
    // second weight set for the fused GeGLU form: y = gelu_tanh(W x) * (W2 x)
    const uint32_t* wq2;
    const uint16_t* scales2;
    const uint16_t* biases2;
    uint32_t* status;
    int64_t N, K;
    int C;        // activation columns = M * split
    int M;        // output rows
    int split;    // columns summed per output row (1 = plain bf16 activations)
    int y_dtype;  // LTHN_DTYPE_*
    int y_split;  // 0: plain y; 2/3: write y as bf16 hi/mid/lo planes ready to be the next qmv's x
    int tma_ok;   // scale/bias tiles may be fetched with bulk copies
};

__device__ __forceinline__ float gelu_tanh_f32(float x) {
    // gelu_tanh as hipGemma4Q4HostGELU (engine/hip/hip_gemma4_q4_layer.go:3582-3597)
    const float k0 = 0.7978845608028654f, k1 = 0.044715f;
    const float inner = k0 * (x + k1 * x * x * x);
    return 0.5f * x * (1.0f + tanhf(inner));
}

// Expand one packed word (8 codes) to four bf16x2 registers holding 128+code:
// p[0]=(c0,c4) p[1]=(c1,c5) p[2]=(c2,c6) p[3]=(c3,c7).
__device__ __forceinline__ void expand_word(uint32_t w, uint32_t (&p)[4]) {
    p[0] = (w & 0x000F000Fu) | 0x43004300u;
    p[1] = ((w >> 4) & 0x000F000Fu) | 0x43004300u;
    p[2] = ((w >> 8) & 0x000F000Fu) | 0x43004300u;
    p[3] = ((w >> 12) & 0x000F000Fu) | 0x43004300u;
}

// Load the 16 activations (bf16, natural order) a lane pairs with its 16 codes
// and permute them to the same (0,4)(1,5)(2,6)(3,7)(8,12).. pairing.
__device__ __forceinline__ void load_x16(const uint16_t* __restrict__ p, uint32_t (&xf)[8]) {
    const uint4 lo = __ldg((const uint4*)p);
    const uint4 hi = __ldg((const uint4*)p + 1);
    xf[0] = __byte_perm(lo.x, lo.z, 0x5410);  // (x0,x4)
    xf[1] = __byte_perm(lo.x, lo.z, 0x7632);  // (x1,x5)
    xf[2] = __byte_perm(lo.y, lo.w, 0x5410);  // (x2,x6)
    xf[3] = __byte_perm(lo.y, lo.w, 0x7632);  // (x3,x7)
    xf[4] = __byte_perm(hi.x, hi.z, 0x5410);
    xf[5] = __byte_perm(hi.x, hi.z, 0x7632);
    xf[6] = __byte_perm(hi.y, hi.w, 0x5410);
    xf[7] = __byte_perm(hi.y, hi.w, 0x7632);
}

// RT: 16-row tiles per CTA (per weight set). NT: 8-column activation tiles.
// FUSE: 0 plain, 1 GeGLU over two weight sets (tile rt of set 1 and of set 2).
// Single-tile, single-column-tile CTAs may be launched with up to 32 (16 when fused) warps so
// that a small matrix has all of its groups in flight at once.
template <int RT, int NT, int FUSE>
__global__ void __launch_bounds__((RT == 1 && NT == 1) ? (FUSE ? 512 : 1024) : 256) qmv_mma_kernel(const QmvArgs a) {
    constexpr int SETS = FUSE == 1 ? 2 : 1;
    constexpr int TR = 16 * RT;  // rows per set per CTA
    extern __shared__ __align__(16) unsigned char smem_raw[];
    __shared__ __align__(8) uint64_t bar;

    pdl_trigger();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    const int qr = lane >> 2, t = lane & 3;
    const int G = (int)(a.K >> 6);
    const int64_t n0 = (int64_t)blockIdx.x * TR;
    const int rows_here = (int)min((int64_t)TR, a.N - n0);

    // shared layout: [SETS][2][TR*G] bf16 scale/bias tiles | reduction | output tile
    uint16_t* sb = (uint16_t*)smem_raw;
    const size_t sb_elems = (size_t)SETS * 2 * TR * G;
    float* red = (float*)(smem_raw + ((sb_elems * 2 + 15) / 16) * 16);

    // ---- stage scale / bias tiles -------------------------------------------
    const bool full = rows_here == TR;
    const bool use_tma = a.tma_ok && full;
    if (use_tma) {
        if (threadIdx.x == 0) {
            mbar_init(&bar, 1);
            mbar_fence_init();
        }
        __syncthreads();
        if (threadIdx.x == 0) {
            const uint32_t bytes = (uint32_t)TR * G * 2;
            mbar_expect_tx(&bar, bytes * 2 * SETS);
            bulk_g2s(sb, a.scales + n0 * G, bytes, &bar);
            bulk_g2s(sb + (size_t)TR * G, a.biases + n0 * G, bytes, &bar);
            if (SETS == 2) {
                bulk_g2s(sb + (size_t)2 * TR * G, a.scales2 + n0 * G, bytes, &bar);
                bulk_g2s(sb + (size_t)3 * TR * G, a.biases2 + n0 * G, bytes, &bar);
            }
        }
    } else {
        const int tile = TR * G;
        for (int i = threadIdx.x; i < tile; i += blockDim.x) {
            const int r = i / G;
            const int64_t src = (n0 + min(r, rows_here - 1)) * G + (i - r * G);
            sb[i] = __ldg(a.scales + src);
            sb[tile + i] = __ldg(a.biases + src);
            if (SETS == 2) {
                sb[2 * tile + i] = __ldg(a.scales2 + src);
                sb[3 * tile + i] = __ldg(a.biases2 + src);
            }
        }
    }

    // rows this lane feeds into the A operand (clamped so tail CTAs stay in bounds)
    const int64_t wpr = a.K >> 3;  // packed words per row
    const uint32_t* wrow[SETS][RT][2];
#pragma unroll
    for (int s = 0; s < SETS; s++)
#pragma unroll
        for (int rt = 0; rt < RT; rt++)
#pragma unroll
            for (int h = 0; h < 2; h++) {
                const int rl = min(16 * rt + qr + 8 * h, rows_here - 1);
                wrow[s][rt][h] = (s == 0 ? a.wq : a.wq2) + (n0 + rl) * wpr + t * 2;
            }
    const uint16_t* xcol[NT];
    bool xlive[NT];
#pragma unroll
    for (int nt = 0; nt < NT; nt++) {
        const int c = nt * 8 + qr;
        xlive[nt] = c < a.C;
        xcol[nt] = a.x + (int64_t)(xlive[nt] ? c : 0) * a.K + t * 16;
    }

    float acc[SETS][RT][NT][4];
#pragma unroll
    for (int s = 0; s < SETS; s++)
#pragma unroll
        for (int rt = 0; rt < RT; rt++)
#pragma unroll
            for (int nt = 0; nt < NT; nt++)
#pragma unroll
                for (int i = 0; i < 4; i++) acc[s][rt][nt][i] = 0.0f;

    // ---- stream the groups this warp owns, one group prefetched ahead -----------
    uint2 wcur[SETS][RT][2], wnxt[SETS][RT][2];
    uint32_t xcur[NT][8], xnxt[NT][8];
    auto load_w = [&](int g, uint2 (&w)[SETS][RT][2]) {
#pragma unroll
        for (int s = 0; s < SETS; s++)
#pragma unroll
            for (int rt = 0; rt < RT; rt++)
#pragma unroll
                for (int h = 0; h < 2; h++) w[s][rt][h] = __ldg((const uint2*)(wrow[s][rt][h] + g * 8));
    };
    auto load_x = [&](int g, uint32_t (&xf)[NT][8]) {
#pragma unroll
        for (int nt = 0; nt < NT; nt++) {
            if (xlive[nt]) {
                load_x16(xcol[nt] + g * 64, xf[nt]);
            } else {
#pragma unroll
                for (int i = 0; i < 8; i++) xf[nt][i] = 0u;
            }
        }
    };

    auto load_group = [&](int g, uint2 (&w)[SETS][RT][2], uint32_t (&xf)[NT][8]) { load_w(g, w); load_x(g, xf); };

    // weights do not depend on the previous kernel: fetch the first group before waiting for it
    int g = warp;
    if (g < G) load_w(g, wcur);
    pdl_wait();
    if (g < G) load_x(g, xcur);

    if (use_tma) {
        if (!mbar_wait(&bar, 0)) {
            if (threadIdx.x == 0) atomicOr(a.status, 1u);
        }
    } else {
        __syncthreads();
    }

    for (; g < G; g += nwarps) {
        const int gn = g + nwarps;
        if (gn < G) load_group(gn, wnxt, xnxt);

        // X_g = sum of the group's activations for this lane's two accumulator columns. The
        // tensor pipe is the scarce resource of this kernel (mma.sync retires one m16n8k16 per
        // ~8 SM cycles on B200), so the sums are formed with f32 adds and shuffles instead of an
        // all-ones MMA in the fused two-weight-set kernel, where the MMA count is highest: each lane
        // adds its 16 values of column qr, the quad completes the group, and the columns 2t and
        // 2t+1 are fetched from the quads that own them. Elsewhere the all-ones MMA is cheaper.
        float xs[NT][2];
        constexpr bool FP_SUMS = FUSE == 1 && NT == 1;  // measured: pays only where the MMA count is highest
#pragma unroll
        for (int nt = 0; nt < NT; nt++) {
            if (FP_SUMS) {
                float part = 0.f;
#pragma unroll
                for (int i = 0; i < 8; i++)
                    part += __uint_as_float(xcur[nt][i] << 16) + __uint_as_float(xcur[nt][i] & 0xffff0000u);
                part += __shfl_xor_sync(0xffffffffu, part, 1);
                part += __shfl_xor_sync(0xffffffffu, part, 2);
                xs[nt][0] = __shfl_sync(0xffffffffu, part, (2 * t) * 4);
                xs[nt][1] = __shfl_sync(0xffffffffu, part, (2 * t + 1) * 4);
            } else {
                // an all-ones A operand yields the sums in exactly the lanes that need them
                float d[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                for (int j = 0; j < 4; j++)
                    mma_bf16_16816(d, 0x3F803F80u, 0x3F803F80u, 0x3F803F80u, 0x3F803F80u, xcur[nt][2 * j], xcur[nt][2 * j + 1]);
                xs[nt][0] = d[0];
                xs[nt][1] = d[1];
            }
        }
#pragma unroll
        for (int s = 0; s < SETS; s++)
#pragma unroll
            for (int rt = 0; rt < RT; rt++) {
                uint32_t pa[8], pb[8];
                {
                    uint32_t q[4];
                    expand_word(wcur[s][rt][0].x, q); pa[0] = q[0]; pa[1] = q[1]; pa[2] = q[2]; pa[3] = q[3];
                    expand_word(wcur[s][rt][0].y, q); pa[4] = q[0]; pa[5] = q[1]; pa[6] = q[2]; pa[7] = q[3];
                    expand_word(wcur[s][rt][1].x, q); pb[0] = q[0]; pb[1] = q[1]; pb[2] = q[2]; pb[3] = q[3];
                    expand_word(wcur[s][rt][1].y, q); pb[4] = q[0]; pb[5] = q[1]; pb[6] = q[2]; pb[7] = q[3];
                }
                const uint16_t* st = sb + (size_t)(2 * s) * TR * G;
                const uint16_t* bt = st + (size_t)TR * G;
                const int ra = (16 * rt + qr) * G + g, rb = ra + 8 * G;
                const float sa = bf16_bits_to_f32(st[ra]), sB = bf16_bits_to_f32(st[rb]);
                const float ca = fmaf(-128.0f, sa, bf16_bits_to_f32(bt[ra]));
                const float cb = fmaf(-128.0f, sB, bf16_bits_to_f32(bt[rb]));
#pragma unroll
                for (int nt = 0; nt < NT; nt++) {
                    float d[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                    for (int j = 0; j < 4; j++)
                        mma_bf16_16816(d, pa[2 * j], pb[2 * j], pa[2 * j + 1], pb[2 * j + 1], xcur[nt][2 * j],
                                       xcur[nt][2 * j + 1]);
                    float* ac = acc[s][rt][nt];
                    ac[0] = fmaf(ca, xs[nt][0], fmaf(sa, d[0], ac[0]));
                    ac[1] = fmaf(ca, xs[nt][1], fmaf(sa, d[1], ac[1]));
                    ac[2] = fmaf(cb, xs[nt][0], fmaf(sB, d[2], ac[2]));
                    ac[3] = fmaf(cb, xs[nt][1], fmaf(sB, d[3], ac[3]));
                }
            }
        if (gn < G) {
#pragma unroll
            for (int s = 0; s < SETS; s++)
#pragma unroll
                for (int rt = 0; rt < RT; rt++) { wcur[s][rt][0] = wnxt[s][rt][0]; wcur[s][rt][1] = wnxt[s][rt][1]; }
#pragma unroll
            for (int nt = 0; nt < NT; nt++)
#pragma unroll
                for (int i = 0; i < 8; i++) xcur[nt][i] = xnxt[nt][i];
        }
    }

    // ---- cross-warp reduction in a fixed order ------------------------------------
    constexpr int PER_WARP = SETS * RT * NT * 128;  // floats each warp contributes
#pragma unroll
    for (int s = 0; s < SETS; s++)
#pragma unroll
        for (int rt = 0; rt < RT; rt++)
#pragma unroll
            for (int nt = 0; nt < NT; nt++)
#pragma unroll
                for (int i = 0; i < 4; i++)
                    red[(size_t)warp * PER_WARP + ((s * RT + rt) * NT + nt) * 128 + i * 32 + lane] = acc[s][rt][nt][i];
    __syncthreads();
    constexpr int CP = NT * 8 + 1;  // padded column stride of the output tile
    float* tile = red + (size_t)nwarps * PER_WARP;  // [SETS][TR][CP]
    for (int e = threadIdx.x; e < PER_WARP; e += blockDim.x) {
        float v = 0.f;
        for (int w = 0; w < nwarps; w++) v += red[(size_t)w * PER_WARP + e];
        const int ln = e & 31, i = (e >> 5) & 3, blk = e >> 7;  // blk = (s*RT+rt)*NT+nt
        const int nt = blk % NT, srt = blk / NT;                // srt = s*RT+rt
        const int s = srt / RT, rt = srt - s * RT;
        const int row = 16 * rt + (ln >> 2) + 8 * (i >> 1);
        const int col = nt * 8 + 2 * (ln & 3) + (i & 1);
        tile[((size_t)s * TR + row) * CP + col] = v;
    }
    __syncthreads();

    // ---- epilogue: add the split columns, optional GeGLU, store --------------------
    for (int e = threadIdx.x; e < a.M * TR; e += blockDim.x) {
        const int m = e / TR, rl = e - m * TR;
        if (rl >= rows_here) continue;
        float v = 0.f;
        for (int j = 0; j < a.split; j++) v += tile[(size_t)rl * CP + m * a.split + j];
        if (FUSE == 1) {
            float u = 0.f;
            for (int j = 0; j < a.split; j++) u += tile[((size_t)TR + rl) * CP + m * a.split + j];
            v = gelu_tanh_f32(v) * u;
        }
        const int64_t n = n0 + rl;
        if (a.y_split > 0) {
            // bf16 hi/mid/lo planes laid out as activation columns m*y_split+j of length N
            uint16_t* yo = (uint16_t*)a.y;
            float r = v;
            for (int j = 0; j < a.y_split; j++) {
                const uint16_t h = f32_to_bf16_bits(r);
                yo[((int64_t)m * a.y_split + j) * a.N + n] = h;
                r -= bf16_bits_to_f32(h);
            }
        } else if (a.y_dtype == LTHN_DTYPE_BF16) {
            ((uint16_t*)a.y)[(int64_t)m * a.N + n] = f32_to_bf16_bits(v);
        } else {
            ((float*)a.y)[(int64_t)m * a.N + n] = v;
        }
    }
}

// ---- f32 -> bf16 column split ---------------------------------------------------
// x f32 [M,K] -> bf16 [M*split, K], column m*split+j = j-th bf16 term of x[m,:]
// (x = hi + mid + lo exactly to 8*split mantissa bits).
__global__ void split_f32_kernel(const float* __restrict__ x, int64_t total, int64_t K, int split,
                                 uint16_t* __restrict__ out) {
    pdl_trigger();
    pdl_wait();
    int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (; i < total; i += stride) {
        const int64_t m = i / K, k = i - m * K;
        float r = x[i];
        for (int j = 0; j < split; j++) {
            const uint16_t h = f32_to_bf16_bits(r);
            out[(m * split + j) * K + k] = h;
            r -= bf16_bits_to_f32(h);
        }
    }
}

// ---- general widths: one warp per output row, SIMT --------------------------------
template <typename XT>
__global__ void qmv_general_kernel(const XT* __restrict__ x, int M, const uint32_t* __restrict__ packed,
                                   const uint16_t* __restrict__ scales, const uint16_t* __restrict__ biases,
                                   int64_t N, int64_t K, int gs, int bits, void* __restrict__ y, int y_dtype) {
    const int lane = threadIdx.x & 31;
    const int64_t row = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= N) return;
    const int epw = 32 / bits;
    const int64_t wpr = K / epw, gpr = K / gs;
    const uint32_t mask = (1u << bits) - 1u;
    for (int m = 0; m < M; m++) {
        float acc = 0.f;
        for (int64_t w = lane; w < wpr; w += 32) {
            const uint32_t word = __ldg(packed + row * wpr + w);
            const int64_t k0 = w * epw;
            for (int p = 0; p < epw; p++) {
                const int64_t k = k0 + p;
                const float s = bf16_bits_to_f32(__ldg(scales + row * gpr + k / gs));
                const float b = bf16_bits_to_f32(__ldg(biases + row * gpr + k / gs));
                const float wv = fmaf(s, (float)((word >> (p * bits)) & mask), b);
                float xv;
                if (sizeof(XT) == 2) xv = bf16_bits_to_f32(((const uint16_t*)x)[(int64_t)m * K + k]);
                else xv = ((const float*)x)[(int64_t)m * K + k];
                acc = fmaf(xv, wv, acc);
            }
        }
        acc = warp_sum(acc);
        if (lane == 0) {
            if (y_dtype == LTHN_DTYPE_BF16) ((uint16_t*)y)[(int64_t)m * N + row] = f32_to_bf16_bits(acc);
            else ((float*)y)[(int64_t)m * N + row] = acc;
        }
    }
}

// ---- host side ------------------------------------------------------------------
static size_t qmv_smem_bytes(int RT, int NT, int sets, int G, int nwarps) {
    const size_t sb = ((size_t)sets * 2 * 16 * RT * G * 2 + 15) / 16 * 16;
    const size_t per_warp = (size_t)sets * RT * NT * 128 * 4;
    const size_t tile = (size_t)sets * 16 * RT * (NT * 8 + 1) * 4;
    return sb + per_warp * nwarps + tile;
}

template <int RT, int NT, int FUSE>
static int32_t launch_one(cudaStream_t s, const QmvArgs& a, int nwarps) {
    const int G = (int)(a.K / 64);
    const size_t smem = qmv_smem_bytes(RT, NT, FUSE == 1 ? 2 : 1, G, nwarps);
    if (smem > 200 * 1024) return fail(LTHN_ERR_INVALID, "affine_qmv: K too large for the shared scale/bias tile");
    static int attr_dev = -1;  // per instantiation
    static std::mutex mu;
    int dev = 0;
    LTHN_CUDA_TRY(cudaGetDevice(&dev));
    {
        std::lock_guard<std::mutex> lk(mu);
        if (attr_dev != dev) {
            LTHN_CUDA_TRY(cudaFuncSetAttribute(qmv_mma_kernel<RT, NT, FUSE>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                               200 * 1024));
            attr_dev = dev;
        }
    }
    const int64_t tr = 16 * RT;
    const unsigned grid = (unsigned)((a.N + tr - 1) / tr);
    LTHN_CUDA_TRY(launch_k(qmv_mma_kernel<RT, NT, FUSE>, dim3(grid), dim3(nwarps * 32), smem, s, a));
    return LTHN_OK;
}

template <int FUSE>
static int32_t launch_qmv(cudaStream_t s, const QmvArgs& a, int rt, int nwarps) {
    const int nt = (a.C + 7) / 8;
#define LTHN_QMV_CASE(R, T) \
    if (rt == R && nt <= T) return launch_one<R, T, FUSE>(s, a, nwarps);
    LTHN_QMV_CASE(1, 1) LTHN_QMV_CASE(2, 1) LTHN_QMV_CASE(4, 1)
    LTHN_QMV_CASE(1, 2) LTHN_QMV_CASE(2, 2) LTHN_QMV_CASE(4, 2)
    LTHN_QMV_CASE(1, 4) LTHN_QMV_CASE(2, 4)
    LTHN_QMV_CASE(1, 8)
    if (nt <= 4) return launch_one<2, 4, FUSE>(s, a, nwarps);
    if (nt <= 8) return launch_one<1, 8, FUSE>(s, a, nwarps);
#undef LTHN_QMV_CASE
    return fail(LTHN_ERR_INVALID, "affine_qmv: more than 64 activation columns");
}

// Picks rows-per-CTA and warps-per-CTA. Small matrices want every SM busy with
// the whole matrix in flight at once (RT=1, many K-splitting warps); large ones
// amortise the activation reads and the epilogue over more rows.
// Tiles per CTA (rt) and K-splitting warps for the bf16 tensor-core kernel, from a sweep on B200
// (f32 activations, C = bf16 columns = rows * split; times for the lm_head / 9216x2304 / 4096x2304
// matrices): long streams want few warps and several tiles per CTA (lm_head, 8 rows: 139 us with
// (4,2) against 230 us with (1,8)); matrices of a few tiles per SM want two tiles and 4-8 warps;
// one tile per SM or less wants every group in flight at once.
void qmv_pick_config(int64_t N, int64_t K, int C, int sets, int* rt, int* nwarps) {
    const int64_t tiles16 = (N + 15) / 16;
    const int G = (int)(K / 64);
    const double tps = (double)tiles16 / 148.0;  // 16-row tiles per SM
    int r = 1, w = 8;
    if (C <= 16) {
        if (tps >= 16.0) { r = 4; w = 2; }
        else if (tps >= 3.0) { r = 2; w = 8; if (sets == 2 && C > 8) { r = 1; w = 4; } }
        else if (C <= 8) {
            // as many K-splitting warps as still let every 16-row tile be resident in one wave
            const int maxw = sets == 2 ? 16 : 32;
            for (int cand = maxw; cand >= 8; cand >>= 1) {
                const int per_sm = std::max(1, std::min(2048 / (32 * cand), 65536 / (80 * 32 * cand)));
                if (tiles16 <= (int64_t)148 * per_sm || cand == 8) { w = cand; break; }
            }
        }
    } else if (C <= 32) {
        if (tps >= 16.0) { r = 2; w = 2; }
        else if (tps >= 3.0) { r = 2; w = 4; }
        else if (tps >= 1.5) { r = 2; w = 8; }
    } else {
        if (tps >= 3.0) w = 2;
        else if (tps >= 1.5) w = 4;
    }
    // the table was measured at K = 2304 (36 groups): keep at most ~18 groups per warp on longer rows
    while (w < 8 && G > 18 * w) w <<= 1;
    if (sets == 2 && r > 2) r = 2;
    while (w > 1 && w > G) w >>= 1;
    *rt = r;
    *nwarps = w;
}

int32_t qmv_launch(cudaStream_t s, QmvArgs a, int fuse, int force_rt, int force_warps) {
    int rt, nwarps;
    qmv_pick_config(a.N, a.K, a.C, fuse == 1 ? 2 : 1, &rt, &nwarps);
    if (force_rt > 0) rt = force_rt;
    if (force_warps > 0) nwarps = force_warps;
    a.status = device_status_word();
    if (!a.status) return fail(LTHN_ERR_CUDA, "affine_qmv: no device status word");
    const int G = (int)(a.K / 64);
    // bulk copies need 16-byte aligned tile starts: tile = 16*rt rows * G * 2 bytes
    a.tma_ok = (((uintptr_t)a.scales | (uintptr_t)a.biases) & 15) == 0 && ((16 * rt * G * 2) % 16) == 0;
    if (fuse == 1) a.tma_ok = a.tma_ok && (((uintptr_t)a.scales2 | (uintptr_t)a.biases2) & 15) == 0;
    if (fuse == 1) return launch_qmv<1>(s, a, rt, nwarps);
    return launch_qmv<0>(s, a, rt, nwarps);
}

int32_t split_f32_launch(cudaStream_t s, const float* x, int64_t M, int64_t K, int split, uint16_t* out) {
    const int64_t total = M * K;
    int grid = (int)std::min<int64_t>((total + 255) / 256, 148 * 8);
    LTHN_CUDA_TRY(launch_k(split_f32_kernel, dim3(grid), dim3(256), 0, s, x, total, K, split, out));
    return LTHN_OK;
}

bool qmv_batch_f32() {
    const char* e = getenv("LTHN_CUDA_BATCH_F32");
    return e && e[0] == '1';
}

// bf16 columns per f32 activation row that producers write for the matvec serving M rows: an
// exact 3-term split at M <= 2, else 2 terms (16 mantissa bits). The tcgen05 kernel reads only the
// first term, which is the bf16 rounding of the value.
int32_t qmv_split_for(int M, int x_dtype) {
    if (x_dtype == LTHN_DTYPE_BF16) return 1;
    return M <= 2 ? 3 : 2;
}

// dispatch overrides: always zero in the product library, which exports no way to set them;
// the test-hook library adds setters (test_hooks.cu)
LTHN_HIDDEN int g_force_rt = 0, g_force_warps = 0, g_force_kernel = 0;

// Routes one call: 1-2 activation rows go to the dp4a kernel, 3..32 rows to the
// tensor-core kernel (f32 activations are first split into bf16 columns).
int32_t qmv_dispatch(cudaStream_t s, const QmvCall& c) {
    const int fuse = c.wq2 ? 1 : 0;
    if (c.bits == 8) {
        // 8-bit codes, one or two rows: the integer tensor-core kernel (plain, GeGLU pair, fused norm prologue)
        I8Plan plan;
        bool aligned = (((uintptr_t)c.wq | (uintptr_t)c.scales | (uintptr_t)c.biases) & 15) == 0;
        if (c.norm) {
            const NormFuse& n = *c.norm;
            aligned = aligned && (((uintptr_t)n.a | (uintptr_t)n.h_in | (uintptr_t)n.h_out | (uintptr_t)n.w_post | (uintptr_t)n.w_next) & 7) == 0;
        } else {
            aligned = aligned && ((uintptr_t)c.x & 15) == 0;
        }
        if (c.wq2) aligned = aligned && (((uintptr_t)c.wq2 | (uintptr_t)c.scales2 | (uintptr_t)c.biases2) & 15) == 0;
        const bool forced = g_force_kernel == 3;
        if (c.M <= 2 && aligned && i8_plan_b8(c.N, c.K, c.M, &plan, forced ? g_force_rt : 0, forced ? g_force_warps : 0, fuse, c.norm != nullptr))
            return i8_launch(s, c, plan);
        return fail(LTHN_ERR_INVALID, "affine_qmv: no integer tensor-core plan for this 8-bit call");
    }
    // Measured on B200: the dp4a kernel wins once a matrix is large enough to amortise its
    // activation conversion (it streams at ~4.5 TB/s where the tensor-core kernel is capped near
    // 3 TB/s by the mma.sync issue rate); small matrices are launch/latency sized and the
    // tensor-core kernel, with every group in flight at once, starts and finishes sooner.
    const double wbytes = (double)c.N * (double)c.K * 0.5625 * (fuse ? 2 : 1);
    const bool big = wbytes >= 28e6 || (wbytes >= 12e6 && c.K >= 4096);
    // Batch 1-2: the integer tensor-core kernel serves every shape it can plan (measured faster than
    // both other kernels from 2 MB matrices to the 340 MB lm_head).
    if ((g_force_kernel == 3 || g_force_kernel == 0) && c.M <= 2) {
        I8Plan plan;
        bool aligned = (((uintptr_t)c.wq | (uintptr_t)c.scales | (uintptr_t)c.biases) & 15) == 0;
        if (c.norm) {
            const NormFuse& n = *c.norm;
            aligned = aligned && (((uintptr_t)n.a | (uintptr_t)n.h_in | (uintptr_t)n.h_out | (uintptr_t)n.w_post | (uintptr_t)n.w_next) & 7) == 0;
        } else {
            aligned = aligned && ((uintptr_t)c.x & 15) == 0;
        }
        if (c.wq2) aligned = aligned && (((uintptr_t)c.wq2 | (uintptr_t)c.scales2 | (uintptr_t)c.biases2) & 15) == 0;
        const bool forced = g_force_kernel == 3;
        if (aligned && i8_plan(c.N, c.K, c.M, fuse, forced ? g_force_rt : 0, forced ? g_force_warps : 0, &plan, (forced && g_force_rt > 1 && !c.norm) ? 8 : 1, c.norm != nullptr))
            return i8_launch(s, c, plan);
        if (forced && g_force_warps) return fail(LTHN_ERR_INVALID, "affine_qmv: forced integer tensor-core configuration is not available");
    }
    if (c.norm) return fail(LTHN_ERR_INVALID, "affine_qmv: a fused norm prologue needs the batch-1/2 integer tensor-core kernel for this shape");
    // 17..32 rows of a large matrix: the tcgen05 streaming kernel (bf16 activations and bf16-rounded
    // weights, the contract of affine_qmm). Measured on B200 against the bf16 mma.sync kernel below:
    // its time does not depend on the row count (lm_head 262144 x 2304: 161 us at 4..32 rows, against
    // 108 / 111 / 143 / 295 / 314 us at 4 / 8 / 16 / 24 / 32 rows; 21504 x 5376: 55 us against 31 / 31 /
    // 46 / 70 / 72 us), so it takes over where the mma.sync kernel runs out of issue slots; matrices
    // of a few MB finish sooner on the mma.sync kernel at every row count.
    const double welems = (double)c.N * (double)c.K * (fuse ? 2 : 1);
    const bool tc_pays = c.M > 16 && welems >= 64e6;
    if (c.M >= 3 && (g_force_kernel == 4 || (g_force_kernel == 0 && tc_pays && !qmv_batch_f32())) && qmv_tc_available(c)) {
        const uint16_t* xb = nullptr;
        int64_t ld = c.K;
        if (c.x_dtype == LTHN_DTYPE_BF16) xb = (const uint16_t*)c.x;
        else if (c.x_cols && c.x_split >= 1) { xb = c.x_cols; ld = (int64_t)c.x_split * c.K; }  // first split term = bf16(x)
        else {
            void* scratch = nullptr;
            int32_t rc = scratch_get((size_t)c.M * c.K * 2, &scratch);
            if (rc) return rc;
            if ((rc = split_f32_launch(s, (const float*)c.x, c.M, c.K, 1, (uint16_t*)scratch))) return rc;
            xb = (const uint16_t*)scratch;
        }
        if (((uintptr_t)xb & 15) == 0) return qmv_tc_launch(s, c, xb, ld);
    }
    const bool prefer_dp4a = g_force_kernel == 1 || (g_force_kernel == 0 && big);
    if (prefer_dp4a && c.M <= 2) {
        Dp4aPlan plan;
        bool aligned = (((uintptr_t)c.wq | (uintptr_t)c.x | (uintptr_t)c.scales | (uintptr_t)c.biases) & 15) == 0;
        if (c.wq2) aligned = aligned && (((uintptr_t)c.wq2 | (uintptr_t)c.scales2 | (uintptr_t)c.biases2) & 15) == 0;
        if (aligned && !(fuse && c.M == 2) && dp4a_plan(c.N, c.K, c.M, fuse, g_force_rt, g_force_warps, &plan))
            return dp4a_launch(s, c, plan);
    }
    QmvArgs a{};
    a.wq = c.wq; a.scales = c.scales; a.biases = c.biases;
    a.wq2 = c.wq2; a.scales2 = c.scales2; a.biases2 = c.biases2;
    a.y = c.y; a.N = c.N; a.K = c.K; a.M = c.M; a.y_dtype = c.y_dtype; a.y_split = 0;
    a.split = c.x_dtype == LTHN_DTYPE_BF16 ? 1 : (c.M <= 2 ? 3 : 2);  // what this kernel wants (see qmv_split_for)
    a.C = c.M * a.split;
    if (c.x_dtype == LTHN_DTYPE_BF16) {
        a.x = (const uint16_t*)c.x;
    } else if (c.x_cols && c.x_split == a.split) {
        a.x = c.x_cols;  // the producer already wrote the bf16 columns
    } else {
        void* scratch = nullptr;
        int32_t rc = scratch_get((size_t)a.C * c.K * 2, &scratch);
        if (rc) return rc;
        rc = split_f32_launch(s, (const float*)c.x, c.M, c.K, a.split, (uint16_t*)scratch);
        if (rc) return rc;
        a.x = (const uint16_t*)scratch;
    }
    const bool cfg = g_force_kernel == 2 || g_force_kernel == 0;
    return qmv_launch(s, a, fuse, cfg ? g_force_rt : 0, cfg ? g_force_warps : 0);
}

}  // namespace lthn

using namespace lthn;

extern "C" {

static int32_t qmv_validate(const void* x, int32_t x_dtype, int32_t M, const void* packed, const void* scales,
                            const void* biases, int64_t N, int64_t K, int32_t gs, int32_t bits, void* y,
                            int32_t y_dtype, cudaStream_t s, bool* done) {
    *done = false;
    LTHN_REQUIRE(M >= 0 && N >= 0 && K >= 0, "affine_qmv: negative dimension");
    if (M == 0 || N == 0) { *done = true; return LTHN_OK; }
    LTHN_REQUIRE(y != nullptr, "affine_qmv: y is NULL");
    LTHN_REQUIRE(x_dtype == LTHN_DTYPE_F32 || x_dtype == LTHN_DTYPE_BF16, "affine_qmv: bad x dtype");
    LTHN_REQUIRE(y_dtype == LTHN_DTYPE_F32 || y_dtype == LTHN_DTYPE_BF16, "affine_qmv: bad y dtype");
    if (K == 0) {
        LTHN_CUDA_TRY(cudaMemsetAsync(y, 0, (size_t)M * N * (y_dtype == LTHN_DTYPE_BF16 ? 2 : 4), s));
        *done = true;
        return LTHN_OK;
    }
    LTHN_REQUIRE(M <= 32, "affine_qmv: M must be at most 32 (use affine_qmm for prefill)");
    LTHN_REQUIRE(bits == 2 || bits == 4 || bits == 8, "affine_qmv: bits must be 2, 4 or 8");
    LTHN_REQUIRE(gs == 32 || gs == 64 || gs == 128, "affine_qmv: group size must be 32, 64 or 128");
    LTHN_REQUIRE(K % gs == 0, "affine_qmv: group size must divide K");
    LTHN_REQUIRE(x && packed && scales && biases, "affine_qmv: NULL pointer");
    return LTHN_OK;
}

int32_t lthn_affine_qmv(void* stream, const void* x, int32_t x_dtype, int32_t M, const uint32_t* packed,
                        const uint16_t* scales, const uint16_t* biases, int64_t N, int64_t K, int32_t gs,
                        int32_t bits, void* y, int32_t y_dtype) {
    clear_error();
    cudaStream_t s = (cudaStream_t)stream;
    bool done = false;
    int32_t rc = qmv_validate(x, x_dtype, M, packed, scales, biases, N, K, gs, bits, y, y_dtype, s, &done);
    if (rc || done) return rc;
    const bool fast = bits == 4 && gs == 64 && ((uintptr_t)packed & 7) == 0 && ((uintptr_t)x & 15) == 0;
    if (bits == 8 && gs == 64 && M <= 2 && (g_force_kernel == 0 || g_force_kernel == 3) && ((uintptr_t)packed & 15) == 0 && ((uintptr_t)x & 15) == 0) {
        // 8-bit codes (the MLP projections of QAT packs): the integer tensor-core kernel takes the bytes as they are
        I8Plan pl;
        if (i8_plan_b8(N, K, M, &pl, g_force_kernel == 3 ? g_force_rt : 0, g_force_kernel == 3 ? g_force_warps : 0)) {
            QmvCall c8{packed, scales, biases, nullptr, nullptr, nullptr, x, x_dtype, y, y_dtype, N, K, M};
            c8.bits = 8;
            return i8_launch(s, c8, pl);
        }
    }
    if (!fast) {
        const int wpb = 8;
        const unsigned grid = (unsigned)((N + wpb - 1) / wpb);
        if (x_dtype == LTHN_DTYPE_BF16)
            qmv_general_kernel<uint16_t><<<grid, wpb * 32, 0, s>>>((const uint16_t*)x, M, packed, scales, biases, N, K, gs, bits, y, y_dtype);
        else
            qmv_general_kernel<float><<<grid, wpb * 32, 0, s>>>((const float*)x, M, packed, scales, biases, N, K, gs, bits, y, y_dtype);
        LTHN_CUDA_TRY(cudaGetLastError());
        return LTHN_OK;
    }
    QmvCall c{packed, scales, biases, nullptr, nullptr, nullptr, x, x_dtype, y, y_dtype, N, K, M};
    return qmv_dispatch(s, c);
}

int32_t lthn_affine_qmv_geglu(void* stream, const void* x, int32_t x_dtype, int32_t M, const uint32_t* gate_packed,
                              const uint16_t* gate_scales, const uint16_t* gate_biases, const uint32_t* up_packed,
                              const uint16_t* up_scales, const uint16_t* up_biases, int64_t N, int64_t K, void* y,
                              int32_t y_dtype) {
    return lthn_affine_qmv_geglu_bits(stream, x, x_dtype, M, gate_packed, gate_scales, gate_biases, up_packed, up_scales, up_biases,
                                      N, K, 4, y, y_dtype);
}

int32_t lthn_affine_qmv_geglu_bits(void* stream, const void* x, int32_t x_dtype, int32_t M, const uint32_t* gate_packed,
                                   const uint16_t* gate_scales, const uint16_t* gate_biases, const uint32_t* up_packed,
                                   const uint16_t* up_scales, const uint16_t* up_biases, int64_t N, int64_t K, int32_t bits,
                                   void* y, int32_t y_dtype) {
    clear_error();
    cudaStream_t s = (cudaStream_t)stream;
    bool done = false;
    LTHN_REQUIRE(bits == 4 || bits == 8, "affine_qmv_geglu: 4-bit or 8-bit codes");
    LTHN_REQUIRE(bits == 4 || M <= 2, "affine_qmv_geglu: 8-bit codes serve one or two rows");
    int32_t rc = qmv_validate(x, x_dtype, M, gate_packed, gate_scales, gate_biases, N, K, 64, bits, y, y_dtype, s, &done);
    if (rc || done) return rc;
    LTHN_REQUIRE(up_packed && up_scales && up_biases, "affine_qmv_geglu: NULL pointer");
    LTHN_REQUIRE(K > 0 && K % 64 == 0, "affine_qmv_geglu: K must be a positive multiple of 64");
    LTHN_REQUIRE((((uintptr_t)gate_packed | (uintptr_t)up_packed) & 7) == 0 && ((uintptr_t)x & 15) == 0,
                 "affine_qmv_geglu: packed weights must be 8-byte and x 16-byte aligned");
    QmvCall c{gate_packed, gate_scales, gate_biases, up_packed, up_scales, up_biases, x, x_dtype, y, y_dtype, N, K, M};
    c.bits = bits;
    return qmv_dispatch(s, c);
}

int32_t lthn_affine_qmv_normed(void* stream, const float* a, const float* h_in, float* h_out, const float* w_post,
                               const float* w_next, float eps, int32_t M, const uint32_t* packed, const uint16_t* scales,
                               const uint16_t* biases, const uint32_t* up_packed, const uint16_t* up_scales,
                               const uint16_t* up_biases, int64_t N, int64_t K, void* y, int32_t y_dtype) {
    return lthn_affine_qmv_normed_bits(stream, a, h_in, h_out, w_post, w_next, eps, M, packed, scales, biases, up_packed, up_scales,
                                       up_biases, N, K, 4, y, y_dtype);
}

int32_t lthn_affine_qmv_normed_bits(void* stream, const float* a, const float* h_in, float* h_out, const float* w_post,
                                    const float* w_next, float eps, int32_t M, const uint32_t* packed, const uint16_t* scales,
                                    const uint16_t* biases, const uint32_t* up_packed, const uint16_t* up_scales,
                                    const uint16_t* up_biases, int64_t N, int64_t K, int32_t bits, void* y, int32_t y_dtype) {
    clear_error();
    LTHN_REQUIRE(bits == 4 || bits == 8, "affine_qmv_normed: 4-bit or 8-bit codes");
    cudaStream_t s = (cudaStream_t)stream;
    LTHN_REQUIRE(M >= 0 && N >= 0 && K >= 0, "affine_qmv_normed: negative dimension");
    if (M == 0 || N == 0) return LTHN_OK;
    LTHN_REQUIRE(M <= 2, "affine_qmv_normed: at most 2 rows");
    LTHN_REQUIRE(h_in && w_next && packed && scales && biases && y, "affine_qmv_normed: NULL pointer");
    LTHN_REQUIRE(!a || (w_post && h_out && h_out != h_in), "affine_qmv_normed: a needs w_post and an h_out that is not h_in");
    LTHN_REQUIRE(K > 0 && K % 64 == 0 && eps >= 0, "affine_qmv_normed: K must be a positive multiple of 64 and eps non-negative");
    LTHN_REQUIRE(y_dtype == LTHN_DTYPE_F32 || y_dtype == LTHN_DTYPE_BF16, "affine_qmv_normed: bad y dtype");
    LTHN_REQUIRE((up_packed == nullptr) == (up_scales == nullptr) && (up_packed == nullptr) == (up_biases == nullptr),
                 "affine_qmv_normed: give all three up_* tensors or none");
    NormFuse nf{a, h_in, h_out, w_post, w_next, eps};
    QmvCall c{packed, scales, biases, up_packed, up_scales, up_biases, nullptr, LTHN_DTYPE_F32, y, y_dtype, N, K, M};
    c.norm = &nf;
    c.bits = bits;
    return qmv_dispatch(s, c);
}

// ---- allocation-free variant ----------------------------------------------------------
// Some hosts must not allocate device memory on the request path: a serving process
// whose memory budget was fixed at start-up (every byte of HBM already handed to the KV
// pool), a caller inside a region where the CUDA allocator may not be entered (a stream
// being captured, a real-time thread), or a sandboxed plugin that is only allowed kernel
// launches. lthn_affine_qmv splits f32 activations into bf16 columns in a scratch buffer
// that it obtains from a growing arena (cudaMalloc on first use or growth); this variant
// keeps that scratch in a fixed array that is part of the loaded module instead.
// The array costs kQmvNoAllocBytes of device memory on every GPU that loads the library,
// for the life of the process.
constexpr size_t kQmvNoAllocBytes = 512u << 10;
constexpr size_t kQmvNoAllocHeader = 256;  // sticky status word, then the bf16 activation columns
static __device__ __align__(256) unsigned char g_qmv_noalloc[kQmvNoAllocBytes];
// g_qmv_noalloc is only a host-side handle here; kernels need the device address, which
// cudaGetSymbolAddress resolves once per device with that device current.
static void* g_qmv_noalloc_addr[16];
static std::mutex g_qmv_noalloc_mu;

int32_t lthn_affine_qmv_noalloc(void* stream, const float* x, int32_t M, const uint32_t* packed,
                                const uint16_t* scales, const uint16_t* biases, int64_t N, int64_t K, float* y) {
    clear_error();
    cudaStream_t s = (cudaStream_t)stream;
    LTHN_REQUIRE(M >= 0 && N >= 0 && K >= 0, "affine_qmv_noalloc: negative dimension");
    if (M == 0 || N == 0) return LTHN_OK;
    LTHN_REQUIRE(x && packed && scales && biases && y, "affine_qmv_noalloc: NULL pointer");
    LTHN_REQUIRE(M <= 32, "affine_qmv_noalloc: M must be at most 32");
    LTHN_REQUIRE(K > 0 && K % 64 == 0, "affine_qmv_noalloc: K must be a positive multiple of 64 (4-bit, group 64 only)");
    LTHN_REQUIRE(((uintptr_t)packed & 7) == 0 && ((uintptr_t)x & 3) == 0, "affine_qmv_noalloc: misaligned pointer");
    const int split = M <= 2 ? 3 : 2;  // the bf16 mma.sync kernel's exact / 16-bit split of f32 activations
    const size_t need = kQmvNoAllocHeader + (size_t)M * split * (size_t)K * 2;
    if (need > kQmvNoAllocBytes)
        return fail(LTHN_ERR_INVALID, "affine_qmv_noalloc: M*" + std::to_string(split) + "*K*2 bytes of activation columns (" +
                                          std::to_string(need - kQmvNoAllocHeader) + ") exceed the fixed scratch of " +
                                          std::to_string(kQmvNoAllocBytes - kQmvNoAllocHeader) +
                                          " bytes; use lthn_affine_qmv for this size");
    int dev = 0;
    LTHN_CUDA_TRY(cudaGetDevice(&dev));
    LTHN_REQUIRE(dev >= 0 && dev < 16, "affine_qmv_noalloc: device index out of range");
    unsigned char* base;
    {
        std::lock_guard<std::mutex> lk(g_qmv_noalloc_mu);
        if (!g_qmv_noalloc_addr[dev]) {  // first call on this device: resolve the array's device address
            void* p = nullptr;
            LTHN_CUDA_TRY(cudaGetSymbolAddress(&p, g_qmv_noalloc));
            // The header's status word must start at zero and is sticky from then on: a kernel
            // whose bounded wait ran out sets a bit that stays until lthn_device_status reads and
            // clears it, so a later call cannot hide an earlier failure.
            LTHN_CUDA_TRY(cudaMemsetAsync(p, 0, kQmvNoAllocHeader, s));
            device_status_register((uint32_t*)p);
            g_qmv_noalloc_addr[dev] = p;
        }
        base = (unsigned char*)g_qmv_noalloc_addr[dev];
    }
    // the array keeps the previous call's bytes; the activation columns are fully rewritten below
    uint16_t* cols = (uint16_t*)(base + kQmvNoAllocHeader);
    int32_t rc = split_f32_launch(s, x, M, K, split, cols);
    if (rc) return rc;
    QmvArgs a{};
    a.wq = packed; a.scales = scales; a.biases = biases; a.x = cols; a.y = y;
    a.N = N; a.K = K; a.M = M; a.C = M * split; a.split = split; a.y_dtype = LTHN_DTYPE_F32; a.y_split = 0;
    a.status = (uint32_t*)base;
    int rt, nwarps;
    qmv_pick_config(N, K, a.C, 1, &rt, &nwarps);
    const int G = (int)(K / 64);
    a.tma_ok = (((uintptr_t)scales | (uintptr_t)biases) & 15) == 0 && ((16 * rt * G * 2) % 16) == 0;
    return launch_qmv<0>(s, a, rt, nwarps);
}

int32_t lthn_affine_qmv_host(const void* x, size_t x_len, const void* packed, size_t packed_len,
                             const void* scales, size_t scales_len, const void* biases, size_t biases_len,
                             int64_t out_dim, int64_t in_dim, int32_t gs, int32_t bits, void* y, size_t y_len) {
    clear_error();
    // validation mirrors enginetest.ReferenceAffineMatVec (quant_reference.go:79-104)
    LTHN_REQUIRE(out_dim >= 0 && in_dim >= 0, "MatVec: outDim/inDim must be non-negative");
    if (out_dim == 0 || in_dim == 0) {
        if (y && y_len >= (size_t)out_dim * 2) memset(y, 0, (size_t)out_dim * 2);
        return LTHN_OK;
    }
    LTHN_REQUIRE(bits > 0 && bits <= 8, "MatVec: bits must be in 1..8");
    LTHN_REQUIRE(gs > 0 && in_dim % gs == 0, "MatVec: groupSize must be > 0 and divide inDim");
    LTHN_REQUIRE((in_dim * bits) % 8 == 0, "MatVec: inDim*bits must be byte-aligned");
    LTHN_REQUIRE(x_len == (size_t)in_dim * 2, "MatVec: len(x) must equal inDim bf16 bytes");
    const size_t row_packed = (size_t)in_dim * bits / 8, row_sb = (size_t)(in_dim / gs) * 2;
    LTHN_REQUIRE(packed_len == out_dim * row_packed && scales_len == out_dim * row_sb && biases_len == out_dim * row_sb,
                 "MatVec: packed/scales/biases size mismatch");
    LTHN_REQUIRE(y_len == (size_t)out_dim * 2, "MatVec: output must hold outDim bf16 values");
    LTHN_REQUIRE(bits == 2 || bits == 4 || bits == 8, "MatVec: this engine serves 2-, 4- and 8-bit affine weights");
    LTHN_REQUIRE(gs == 32 || gs == 64 || gs == 128, "MatVec: this engine serves group sizes 32, 64 and 128");
    LTHN_REQUIRE((in_dim * bits) % 32 == 0, "MatVec: inDim*bits must fill whole 32-bit words");

    // The staging arena (slot 1) and the stream are shared by every caller: concurrent MatVec calls
    // from several host threads take turns here.
    static std::mutex host_mu;
    std::lock_guard<std::mutex> host_lk(host_mu);
    // one allocation, 256-byte aligned sections
    auto up = [](size_t v) { return (v + 255) / 256 * 256; };
    const size_t o_x = 0, o_p = o_x + up(x_len), o_s = o_p + up(packed_len), o_b = o_s + up(scales_len),
                 o_y = o_b + up(biases_len), total = o_y + up(y_len);
    unsigned char* d = nullptr;
    {
        void* arena = nullptr;
        int32_t arc = scratch_get(total, &arena, 1);  // cached staging arena: no cudaMalloc per call
        if (arc) return arc;
        d = (unsigned char*)arena;
    }
    cudaStream_t s = nullptr;
    int32_t rc = LTHN_OK;
    cudaError_t e;
    if ((e = cudaMemcpyAsync(d + o_x, x, x_len, cudaMemcpyHostToDevice, s)) != cudaSuccess ||
        (e = cudaMemcpyAsync(d + o_p, packed, packed_len, cudaMemcpyHostToDevice, s)) != cudaSuccess ||
        (e = cudaMemcpyAsync(d + o_s, scales, scales_len, cudaMemcpyHostToDevice, s)) != cudaSuccess ||
        (e = cudaMemcpyAsync(d + o_b, biases, biases_len, cudaMemcpyHostToDevice, s)) != cudaSuccess) {
        rc = cuda_fail(e, "MatVec: host to device copy");
    }
    if (rc == LTHN_OK)
        rc = lthn_affine_qmv(s, d + o_x, LTHN_DTYPE_BF16, 1, (const uint32_t*)(d + o_p), (const uint16_t*)(d + o_s),
                             (const uint16_t*)(d + o_b), out_dim, in_dim, gs, bits, d + o_y, LTHN_DTYPE_BF16);
    if (rc == LTHN_OK && (e = cudaMemcpyAsync(y, d + o_y, y_len, cudaMemcpyDeviceToHost, s)) != cudaSuccess)
        rc = cuda_fail(e, "MatVec: device to host copy");
    if (rc == LTHN_OK && (e = cudaStreamSynchronize(s)) != cudaSuccess) rc = cuda_fail(e, "MatVec: synchronize");
    if (rc == LTHN_OK) rc = check_device_status(s);
    return rc;
}

}  // extern "C"
