// qmm.cu — affine_qmm: prefill-time MLX-affine 4-bit matmul on the Blackwell
// tensor cores (tcgen05.mma, accumulators in TMEM), written for B200 (sm_100a).
//
//   Y[M,N] (bf16) = X[M,K] (bf16) * dequant(W[N,K])^T,  fp32 accumulation.
//
// One CTA computes a 256-token x NT-row output tile (NT = 128 or 256) and is
// warp-specialised around a ring of shared-memory stages, each holding one
// k-block of 64 (= one quantisation group = one 128-byte swizzle row of bf16):
//
//   warp 0      TMA producer: cp.async.bulk.tensor loads the X tile (256 x 64 bf16,
//               128-byte swizzle) of a stage, completing on the stage's mbarrier.
//   warp 1      MMA issuer: one elected lane issues 2 x 4 tcgen05.mma (M=128, N=NT,
//               K=16, bf16 x bf16 -> f32) per k-block into two TMEM accumulators
//               (token rows 0-127 and 128-255), then tcgen05.commit frees the stage.
//               It also owns the TMEM allocation.
//   warps 2-9   dequantisers: read the packed codes and the bf16 scale/bias of their
//               rows, expand codes to bf16 with one logic op per pair
//               ((w>>4i & 0x000F000F) | 0x43004300 = {128+q, 128+q'}), subtract 128
//               and apply w = scale*q + bias in one bf16x2 FMA (a single rounding of
//               the exact value), and store the 64-wide row slice into the stage in
//               the same swizzled K-major layout TMA produces. After the K loop they
//               become the epilogue: tcgen05.ld the accumulators, round to bf16, store.
//
// Dequantising the W tile costs about 2.5 issue slots per weight element while the
// tensor cores spend 1024 cycles on a 256x256x64 k-block, so the dequantisers use about
// a third of the SM's issue rate and stay ahead of the MMA pipe; the kernel is bound by
// tensor throughput. Every mbarrier wait is bounded: on a time-out the kernel records it
// in the device status word, releases its TMEM and returns.
#include "common.cuh"
#include "qmv.hpp"

#include <cuda.h>

#include <algorithm>
#include <mutex>

namespace lthn {

constexpr int QMM_BK = 64;
constexpr int QMM_MT = 256;  // tokens per CTA tile (two 128-row accumulators)
constexpr int QMM_DQ_THREADS = 256;
constexpr int QMM_THREADS = 64 + QMM_DQ_THREADS;

template <int NT>
struct QmmSmem {
    static constexpr int STAGES = NT == 256 ? 3 : 4;
    static constexpr int X_BYTES = QMM_MT * QMM_BK * 2;  // 32 KB
    static constexpr int W_BYTES = NT * QMM_BK * 2;      // 32 / 16 KB
    static constexpr int STAGE_BYTES = X_BYTES + W_BYTES;
    static constexpr int TOTAL = STAGES * STAGE_BYTES + 1024 /*alignment slack*/ + 256 /*barriers*/;
};

struct QmmArgs {
    const uint32_t* wq;
    const uint16_t* scales;
    const uint16_t* biases;
    // GeGLU pair (wq2 != NULL): a CTA's weight tile holds NT/2 rows of the gate matrix followed by
    // the same NT/2 rows of the up matrix, and the epilogue stores gelu_tanh(gate) * up
    const uint32_t* wq2;
    const uint16_t* scales2;
    const uint16_t* biases2;
    void* y;       // [M, N] bf16, or f32 when y_f32
    uint32_t* status;
    int M, N, K;   // N = output columns
    int y_f32;
    // split-K (gridDim.z > 1): CTA z works on k-blocks [z*kb_per, (z+1)*kb_per) and stores its f32 partial
    // sums at y + z*M*N; a second kernel adds the partials
    int kb_per;
};

// ---- tcgen05 / TMA wrappers -----------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_dst, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_dst)), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

__device__ __forceinline__ void umma_bf16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int c0, int c1, uint64_t* bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 ::"r"(smem_u32(dst)), "l"(map), "r"(c0), "r"(c1), "r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// K-major, 128-byte swizzle, 8-row groups 1024 bytes apart (tile base 1024-aligned)
__device__ __forceinline__ uint64_t umma_desc(uint32_t smem_addr) {
    return (uint64_t)((smem_addr & 0x3FFFFu) >> 4) | ((uint64_t)1 << 16) | ((uint64_t)(1024 >> 4) << 32) |
           ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
}

__device__ __forceinline__ uint32_t bf16x2_sub(uint32_t a, uint32_t b) {
    uint32_t d;
    asm("sub.rn.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
    return d;
}
__device__ __forceinline__ uint32_t bf16x2_fma(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t d;
    asm("fma.rn.bf16x2 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}

// 8 codes of one packed word -> 8 bf16 weights in memory order (one 16-byte chunk)
__device__ __forceinline__ uint4 dequant_word(uint32_t w, uint32_t s2, uint32_t b2) {
    const uint32_t k128 = 0x43004300u;
    uint32_t p0 = (w & 0x000F000Fu) | k128;          // (c0, c4) + 128
    uint32_t p1 = ((w >> 4) & 0x000F000Fu) | k128;   // (c1, c5)
    uint32_t p2 = ((w >> 8) & 0x000F000Fu) | k128;   // (c2, c6)
    uint32_t p3 = ((w >> 12) & 0x000F000Fu) | k128;  // (c3, c7)
    p0 = bf16x2_fma(bf16x2_sub(p0, k128), s2, b2);
    p1 = bf16x2_fma(bf16x2_sub(p1, k128), s2, b2);
    p2 = bf16x2_fma(bf16x2_sub(p2, k128), s2, b2);
    p3 = bf16x2_fma(bf16x2_sub(p3, k128), s2, b2);
    uint4 o;
    o.x = __byte_perm(p0, p1, 0x5410);  // (w0, w1)
    o.y = __byte_perm(p2, p3, 0x5410);  // (w2, w3)
    o.z = __byte_perm(p0, p1, 0x7632);  // (w4, w5)
    o.w = __byte_perm(p2, p3, 0x7632);  // (w6, w7)
    return o;
}

// 8-bit codes: 8 codes of two packed words -> 8 bf16 weights in memory order. A byte is hi*16 + lo with both
// nibbles exact in bf16 and so is their sum (8 significant bits), so scale*q + bias is rounded once, as for 4 bits.
__device__ __forceinline__ void dequant_half8(uint32_t w, uint32_t s2, uint32_t b2, uint32_t& o01, uint32_t& o23) {
    const uint32_t k128 = 0x43004300u, k16 = 0x41804180u;
    const uint32_t lo02 = bf16x2_sub((w & 0x000F000Fu) | k128, k128), hi02 = bf16x2_sub(((w >> 4) & 0x000F000Fu) | k128, k128);
    const uint32_t lo13 = bf16x2_sub(((w >> 8) & 0x000F000Fu) | k128, k128), hi13 = bf16x2_sub(((w >> 12) & 0x000F000Fu) | k128, k128);
    const uint32_t p02 = bf16x2_fma(bf16x2_fma(hi02, k16, lo02), s2, b2);  // (c0, c2)
    const uint32_t p13 = bf16x2_fma(bf16x2_fma(hi13, k16, lo13), s2, b2);  // (c1, c3)
    o01 = __byte_perm(p02, p13, 0x5410);
    o23 = __byte_perm(p02, p13, 0x7632);
}
__device__ __forceinline__ uint4 dequant_words8(uint32_t w0, uint32_t w1, uint32_t s2, uint32_t b2) {
    uint4 o;
    dequant_half8(w0, s2, b2, o.x, o.y);
    dequant_half8(w1, s2, b2, o.z, o.w);
    return o;
}

__device__ __forceinline__ float qmm_gelu_tanh(float x) {
    // gelu_tanh as hipGemma4Q4HostGELU (engine/hip/hip_gemma4_q4_layer.go:3582-3597)
    const float k0 = 0.7978845608028654f, k1 = 0.044715f;
    return 0.5f * x * (1.0f + tanhf(k0 * (x + k1 * x * x * x)));
}

// GEGLU: 0 plain, 1 gate/up pair (see QmmArgs). BITS: 4, or 8 (one code per byte).
template <int NT, int GEGLU, int BITS>
__global__ void __launch_bounds__(QMM_THREADS, 1)
qmm_tcgen05_kernel(const __grid_constant__ CUtensorMap x_map, const QmmArgs a) {
    using S = QmmSmem<NT>;
    constexpr int NO = GEGLU ? NT / 2 : NT;   // output columns per CTA
    constexpr int STAGES = S::STAGES;
    constexpr int TPR = QMM_DQ_THREADS / NT;  // dequant threads per weight row: 1 (NT=256) or 2 (NT=128)
    constexpr int WPG = BITS * 2;             // packed words per group and row: 8 or 16
    constexpr int WORDS = WPG / TPR;          // of them per thread
    constexpr int CHUNKS = 8 / TPR;           // 16-byte chunks (8 bf16 weights) a thread writes per k-block
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = (unsigned char*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint64_t* bars = (uint64_t*)(smem + STAGES * S::STAGE_BYTES);
    uint64_t* full_x = bars;
    uint64_t* full_w = bars + STAGES;
    uint64_t* empty = bars + 2 * STAGES;
    uint64_t* accum_full = bars + 3 * STAGES;
    uint32_t* tmem_slot = (uint32_t*)(bars + 3 * STAGES + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n0 = blockIdx.x * NO, m0 = blockIdx.y * QMM_MT;
    const int KB = a.K / QMM_BK;
    const int kb_lo = gridDim.z > 1 ? (int)blockIdx.z * a.kb_per : 0;
    const int kb_hi = gridDim.z > 1 ? min(KB, kb_lo + a.kb_per) : KB;
    bool ok = true;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; s++) {
            mbar_init(&full_x[s], 1);
            mbar_init(&full_w[s], QMM_DQ_THREADS);
            mbar_init(&empty[s], 1);
        }
        mbar_init(accum_full, 1);
        mbar_fence_init();
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, 2 * NT);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ---- TMA producer ------------------------------------------------------------
        if (lane == 0) {
            for (int kb = kb_lo; kb < kb_hi && ok; kb++) {
                const int s = (kb - kb_lo) % STAGES, ph = ((kb - kb_lo) / STAGES) & 1;
                ok = mbar_wait(&empty[s], ph ^ 1);
                if (!ok) break;
                mbar_expect_tx(&full_x[s], S::X_BYTES);
                tma_load_2d(smem + s * S::STAGE_BYTES, &x_map, kb * QMM_BK, m0, &full_x[s]);
            }
            if (!ok) atomicOr(a.status, 2u);
        }
    } else if (warp == 1) {
        // ---- MMA issuer ----------------------------------------------------------------
        if (lane == 0) {
            const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(NT >> 3) << 17) | ((128u >> 4) << 24);
            for (int kb = kb_lo; kb < kb_hi && ok; kb++) {
                const int s = (kb - kb_lo) % STAGES, ph = ((kb - kb_lo) / STAGES) & 1;
                ok = mbar_wait(&full_x[s], ph) && mbar_wait(&full_w[s], ph);
                if (!ok) break;
                tc_fence_after();
                const uint32_t xs = smem_u32(smem + s * S::STAGE_BYTES);
                const uint32_t ws = xs + S::X_BYTES;
#pragma unroll
                for (int h = 0; h < 2; h++)
#pragma unroll
                    for (int j = 0; j < 4; j++)
                        umma_bf16(tmem_base + h * NT, umma_desc(xs + h * 128 * 128 + j * 32), umma_desc(ws + j * 32), idesc,
                                  (kb > kb_lo || j > 0) ? 1u : 0u);
                umma_commit(&empty[s]);
            }
            if (ok) umma_commit(accum_full);
            else atomicOr(a.status, 4u);
        }
    } else {
        // ---- dequantisers, then epilogue -------------------------------------------------
        const int t = threadIdx.x - 64;
        const int row = t / TPR, part = t - row * TPR;
        const bool second = GEGLU && row >= NO;       // tile rows NO.. come from the up matrix
        const int64_t grow = min(n0 + (second ? row - NO : row), a.N - 1);  // tail tiles re-read the last row; never stored
        const uint32_t* wp = (second ? a.wq2 : a.wq) + grow * ((int64_t)a.K * BITS / 32) + part * WORDS;
        const uint16_t* sp = (second ? a.scales2 : a.scales) + grow * KB;
        const uint16_t* bp = (second ? a.biases2 : a.biases) + grow * KB;
        uint32_t wcur[WORDS], wnxt[WORDS];
        uint32_t sbcur, sbnxt = 0;
        auto load_kb = [&](int kb, uint32_t (&w)[WORDS], uint32_t& sb) {
#pragma unroll
            for (int v = 0; v < WORDS / 4; v++) {
                const uint4 q = __ldg((const uint4*)(wp + (int64_t)kb * WPG) + v);
                w[4 * v] = q.x; w[4 * v + 1] = q.y; w[4 * v + 2] = q.z; w[4 * v + 3] = q.w;
            }
            sb = (uint32_t)__ldg(sp + kb) | ((uint32_t)__ldg(bp + kb) << 16);
        };
        load_kb(kb_lo, wcur, sbcur);
        for (int kb = kb_lo; kb < kb_hi && ok; kb++) {
            const int s = (kb - kb_lo) % STAGES, ph = ((kb - kb_lo) / STAGES) & 1;
            if (kb + 1 < kb_hi) load_kb(kb + 1, wnxt, sbnxt);
            ok = mbar_wait(&empty[s], ph ^ 1);
            if (!ok) break;
            const uint32_t s2 = (sbcur & 0xffffu) | (sbcur << 16);
            const uint32_t b2 = (sbcur >> 16) | (sbcur & 0xffff0000u);
            unsigned char* wrow = smem + s * S::STAGE_BYTES + S::X_BYTES + row * 128;
#pragma unroll
            for (int i = 0; i < CHUNKS; i++) {
                const int c = part * CHUNKS + i;  // 16-byte chunk index within the 128-byte row
                uint4 o;
                if constexpr (BITS == 8) o = dequant_words8(wcur[(2 * i) % WORDS], wcur[(2 * i + 1) % WORDS], s2, b2);
                else o = dequant_word(wcur[i % WORDS], s2, b2);
                *(uint4*)(wrow + ((c ^ (row & 7)) << 4)) = o;
            }
            fence_async_smem();
            mbar_arrive(&full_w[s]);
#pragma unroll
            for (int i = 0; i < WORDS; i++) wcur[i] = wnxt[i];
            sbcur = sbnxt;
        }
        if (!ok) atomicOr(a.status, 8u);
        // epilogue: warp w may touch TMEM lanes 32*(w%4)..+31; warps 2-5 take accumulator 0, 6-9 accumulator 1
        if (ok) ok = mbar_wait(accum_full, 0);
        if (ok) {
            tc_fence_after();
            const int quad = warp & 3, half = (warp - 2) >> 2;
            const int m = m0 + half * 128 + quad * 32 + lane;
            const uint32_t tbase = tmem_base + ((uint32_t)(quad * 32) << 16) + half * NT;
#pragma unroll 1
            for (int c0 = 0; c0 < NO; c0 += 32) {
                uint32_t r[32];
                tmem_ld32(tbase + c0, r);
                if (GEGLU) {
                    uint32_t u[32];
                    tmem_ld32(tbase + NO + c0, u);
                    tmem_ld_wait();
#pragma unroll
                    for (int e = 0; e < 32; e++)
                        r[e] = __float_as_uint(qmm_gelu_tanh(__uint_as_float(r[e])) * __uint_as_float(u[e]));
                } else {
                    tmem_ld_wait();
                }
                if (m < a.M) {
                    if (a.y_f32) {
                        float* yrow = (float*)a.y + (gridDim.z > 1 ? (int64_t)blockIdx.z * a.M * a.N : 0) + (int64_t)m * a.N + n0 + c0;
                        if (n0 + c0 + 32 <= a.N && (((uintptr_t)yrow) & 15) == 0) {
#pragma unroll
                            for (int v = 0; v < 8; v++)
                                *(uint4*)(yrow + v * 4) = make_uint4(r[v * 4], r[v * 4 + 1], r[v * 4 + 2], r[v * 4 + 3]);
                        } else {
                            for (int e = 0; e < 32; e++)
                                if (n0 + c0 + e < a.N) yrow[e] = __uint_as_float(r[e]);
                        }
                        continue;
                    }
                    uint16_t* yrow = (uint16_t*)a.y + (int64_t)m * a.N + n0 + c0;
                    if (n0 + c0 + 32 <= a.N && (((uintptr_t)yrow) & 15) == 0) {
#pragma unroll
                        for (int v = 0; v < 4; v++) {
                            uint4 o;
                            uint32_t* po = (uint32_t*)&o;
#pragma unroll
                            for (int e = 0; e < 4; e++)
                                po[e] = (uint32_t)f32_to_bf16_bits(__uint_as_float(r[v * 8 + 2 * e])) |
                                        ((uint32_t)f32_to_bf16_bits(__uint_as_float(r[v * 8 + 2 * e + 1])) << 16);
                            *(uint4*)(yrow + v * 8) = o;
                        }
                    } else {
                        for (int e = 0; e < 32; e++)
                            if (n0 + c0 + e < a.N) yrow[e] = f32_to_bf16_bits(__uint_as_float(r[e]));
                    }
                }
            }
        } else {
            atomicOr(a.status, 16u);
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem_base, 2 * NT);
}

// ---- host side -----------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)p;
    }
    return fn;
}

// adds the split-K partial sums [splits][n] (f32) in split order; out: f32 or bf16
__global__ void qmm_splitk_sum_kernel(const float* __restrict__ part, int splits, int64_t n, void* __restrict__ out, int out_f32) {
    const int64_t i = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) * 4;
    if (i >= n) return;
    float4 acc = *(const float4*)(part + i);
    for (int z = 1; z < splits; z++) {
        const float4 v = *(const float4*)(part + (int64_t)z * n + i);
        acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
    }
    if (out_f32) {
        *(float4*)((float*)out + i) = acc;
    } else {
        uint2 o;
        o.x = (uint32_t)f32_to_bf16_bits(acc.x) | ((uint32_t)f32_to_bf16_bits(acc.y) << 16);
        o.y = (uint32_t)f32_to_bf16_bits(acc.z) | ((uint32_t)f32_to_bf16_bits(acc.w) << 16);
        *(uint2*)((uint16_t*)out + i) = o;
    }
}

template <int NT, int GEGLU, int BITS>
static int32_t launch_qmm_b(cudaStream_t s, const CUtensorMap& map, const QmmArgs& a, int splits) {
    static int attr_dev = -1;
    static std::mutex mu;
    int dev = 0;
    LTHN_CUDA_TRY(cudaGetDevice(&dev));
    {
        std::lock_guard<std::mutex> lk(mu);
        if (attr_dev != dev) {
            LTHN_CUDA_TRY(cudaFuncSetAttribute(qmm_tcgen05_kernel<NT, GEGLU, BITS>, cudaFuncAttributeMaxDynamicSharedMemorySize, QmmSmem<NT>::TOTAL));
            attr_dev = dev;
        }
    }
    constexpr int NO = GEGLU ? NT / 2 : NT;
    dim3 grid((a.N + NO - 1) / NO, (a.M + QMM_MT - 1) / QMM_MT, splits);
    qmm_tcgen05_kernel<NT, GEGLU, BITS><<<grid, QMM_THREADS, QmmSmem<NT>::TOTAL, s>>>(map, a);
    LTHN_CUDA_TRY(cudaGetLastError());
    return LTHN_OK;
}
template <int NT, int GEGLU>
static int32_t launch_qmm(cudaStream_t s, const CUtensorMap& map, const QmmArgs& a, int bits, int splits = 1) {
    return bits == 8 ? launch_qmm_b<NT, GEGLU, 8>(s, map, a, splits) : launch_qmm_b<NT, GEGLU, 4>(s, map, a, splits);
}

LTHN_HIDDEN int g_force_nt = 0;  // tile override: zero in the product library (setter: test_hooks.cu)

// The tensor-core path for any M >= 1 (rows past M are zero-filled by the TMA load and never
// stored): 4-bit or 8-bit codes, group 64, x and packed 16-byte aligned.
int32_t qmm_launch(cudaStream_t s, const QmmCall& c) {
    if (!encode_fn()) return fail(LTHN_ERR_UNAVAILABLE, "affine_qmm: cuTensorMapEncodeTiled is not available from this driver");
    CUtensorMap map;
    const cuuint64_t dims[2] = {(cuuint64_t)c.K, (cuuint64_t)c.M};
    const cuuint64_t strides[1] = {(cuuint64_t)c.K * 2};
    const cuuint32_t box[2] = {QMM_BK, QMM_MT};
    const cuuint32_t estr[2] = {1, 1};
    CUresult cr = encode_fn()(&map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (void*)c.x, dims, strides, box, estr,
                              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (cr != CUDA_SUCCESS) return fail(LTHN_ERR_CUDA, "affine_qmm: cuTensorMapEncodeTiled failed (" + std::to_string((int)cr) + ")");
    QmmArgs a{c.wq, c.scales, c.biases, c.wq2, c.scales2, c.biases2, c.y, device_status_word(), c.M, (int)c.N, (int)c.K, c.y_f32, 0};
    if (!a.status) return fail(LTHN_ERR_CUDA, "affine_qmm: no device status word");
    const int64_t mt = (c.M + QMM_MT - 1) / QMM_MT;
    // Tile width by wave efficiency: one CTA per SM, so a grid of T tiles takes ceil(T/SMs) waves
    // and the last wave may be nearly empty (N = 5376 with 2048 tokens is 168 tiles of 256 =
    // 1.13 waves). The narrower tile does the same work in more, smaller pieces, at about 0.9 of
    // the wide tile's rate per SM (measured ratio at full waves).
    int sms = 148;
    {
        int dev = 0;
        if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    }
    auto eff = [&](int64_t tiles) { return (double)tiles / (double)(((tiles + sms - 1) / sms) * sms); };
    const int no256 = c.wq2 ? 128 : 256, no128 = c.wq2 ? 64 : 128;  // output columns per tile (a GeGLU tile is half gate, half up)
    const double e256 = eff(((c.N + no256 - 1) / no256) * mt), e128 = 0.9 * eff(((c.N + no128 - 1) / no128) * mt);
    int nt = e256 >= e128 ? 256 : 128;
    if (g_force_nt == 128 || g_force_nt == 256) nt = g_force_nt;
    if (c.bits != 4 && c.bits != 8) return fail(LTHN_ERR_INVALID, "affine_qmm: the tensor-core kernel reads 4-bit or 8-bit codes");
    if (c.wq2) return nt == 256 ? launch_qmm<256, 1>(s, map, a, c.bits) : launch_qmm<128, 1>(s, map, a, c.bits);
    // Split-K when the output has too few tiles to fill the GPU (the long-K, narrow projections of a
    // short prompt: 2304 x 9216 with 512 tokens is 36 tiles): z CTAs per tile each take a slice of at
    // least 16 k-blocks and leave f32 partial sums that a second kernel adds in slice order.
    const int64_t tiles = ((c.N + (nt == 256 ? 256 : 128) - 1) / (nt == 256 ? 256 : 128)) * mt;
    const int KB = (int)(c.K / QMM_BK);
    int splits = (int)std::min<int64_t>({4, sms / std::max<int64_t>(tiles, 1), KB / 16});
    if (splits >= 2 && ((int64_t)c.M * c.N) % 4 == 0) {
        a.kb_per = (KB + splits - 1) / splits;
        splits = (KB + a.kb_per - 1) / a.kb_per;
        void* part = nullptr;
        int32_t rc;
        if ((rc = scratch_get((size_t)splits * c.M * c.N * sizeof(float), &part, 0))) return rc;
        QmmArgs pa = a;
        pa.y = part;
        pa.y_f32 = 1;
        if ((rc = nt == 256 ? launch_qmm<256, 0>(s, map, pa, c.bits, splits) : launch_qmm<128, 0>(s, map, pa, c.bits, splits))) return rc;
        const int64_t n = (int64_t)c.M * c.N;
        qmm_splitk_sum_kernel<<<(unsigned)((n / 4 + 255) / 256), 256, 0, s>>>((const float*)part, splits, n, c.y, c.y_f32);
        LTHN_CUDA_TRY(cudaGetLastError());
        return LTHN_OK;
    }
    return nt == 256 ? launch_qmm<256, 0>(s, map, a, c.bits) : launch_qmm<128, 0>(s, map, a, c.bits);
}

}  // namespace lthn

using namespace lthn;

extern "C" {

int32_t lthn_affine_qmm(void* stream, const uint16_t* x, int32_t M, const uint32_t* packed, const uint16_t* scales,
                        const uint16_t* biases, int64_t N, int64_t K, int32_t gs, int32_t bits, uint16_t* y) {
    clear_error();
    cudaStream_t s = (cudaStream_t)stream;
    LTHN_REQUIRE(M >= 0 && N >= 0 && K >= 0, "affine_qmm: negative dimension");
    if (M == 0 || N == 0) return LTHN_OK;
    LTHN_REQUIRE(y != nullptr, "affine_qmm: y is NULL");
    if (K == 0) {
        LTHN_CUDA_TRY(cudaMemsetAsync(y, 0, (size_t)M * N * 2, s));
        return LTHN_OK;
    }
    LTHN_REQUIRE(x && packed && scales && biases, "affine_qmm: NULL pointer");
    LTHN_REQUIRE(bits == 2 || bits == 4 || bits == 8, "affine_qmm: bits must be 2, 4 or 8");
    LTHN_REQUIRE(gs == 32 || gs == 64 || gs == 128, "affine_qmm: group size must be 32, 64 or 128");
    LTHN_REQUIRE(K % gs == 0, "affine_qmm: group size must divide K");
    LTHN_REQUIRE(N < (int64_t)1 << 31 && K < (int64_t)1 << 31, "affine_qmm: dimension too large");
    const bool tensor_path = (bits == 4 || bits == 8) && gs == 64 && M > 32 && (((uintptr_t)x | (uintptr_t)packed) & 15) == 0 && encode_fn();
    if (!tensor_path) {
        // small M and the other widths of the format: the decode kernels, 32 rows at a time
        for (int m0 = 0; m0 < M; m0 += 32) {
            const int rows = std::min(32, M - m0);
            int32_t rc = lthn_affine_qmv(stream, x + (int64_t)m0 * K, LTHN_DTYPE_BF16, rows, packed, scales, biases, N, K, gs,
                                         bits, y + (int64_t)m0 * N, LTHN_DTYPE_BF16);
            if (rc) return rc;
        }
        return LTHN_OK;
    }
    QmmCall c{x, M, packed, scales, biases, nullptr, nullptr, nullptr, N, K, y, 0};
    c.bits = bits;
    return qmm_launch(s, c);
}

int32_t lthn_affine_qmm_geglu(void* stream, const uint16_t* x, int32_t M, const uint32_t* gate_packed,
                              const uint16_t* gate_scales, const uint16_t* gate_biases, const uint32_t* up_packed,
                              const uint16_t* up_scales, const uint16_t* up_biases, int64_t N, int64_t K, uint16_t* y) {
    return lthn_affine_qmm_geglu_bits(stream, x, M, gate_packed, gate_scales, gate_biases, up_packed, up_scales, up_biases, N, K, 4, y);
}

int32_t lthn_affine_qmm_geglu_bits(void* stream, const uint16_t* x, int32_t M, const uint32_t* gate_packed,
                                   const uint16_t* gate_scales, const uint16_t* gate_biases, const uint32_t* up_packed,
                                   const uint16_t* up_scales, const uint16_t* up_biases, int64_t N, int64_t K, int32_t bits,
                                   uint16_t* y) {
    clear_error();
    LTHN_REQUIRE(bits == 4 || bits == 8, "affine_qmm_geglu: 4-bit or 8-bit codes");
    LTHN_REQUIRE(M >= 0 && N >= 0 && K >= 0, "affine_qmm_geglu: negative dimension");
    if (M == 0 || N == 0) return LTHN_OK;
    LTHN_REQUIRE(x && gate_packed && gate_scales && gate_biases && up_packed && up_scales && up_biases && y,
                 "affine_qmm_geglu: NULL pointer");
    LTHN_REQUIRE(K > 0 && K % 64 == 0, "affine_qmm_geglu: K must be a positive multiple of 64 (group 64 only)");
    LTHN_REQUIRE(N < (int64_t)1 << 31 && K < (int64_t)1 << 31, "affine_qmm_geglu: dimension too large");
    LTHN_REQUIRE((((uintptr_t)x | (uintptr_t)gate_packed | (uintptr_t)up_packed) & 15) == 0,
                 "affine_qmm_geglu: x and the packed weights must be 16-byte aligned");
    QmmCall c{x, M, gate_packed, gate_scales, gate_biases, up_packed, up_scales, up_biases, N, K, y, 0};
    c.bits = bits;
    return qmm_launch((cudaStream_t)stream, c);
}

}  // extern "C"
