// qmv_tc.cu — affine_qmv for 3..32 activation rows on the Blackwell tensor cores
// (tcgen05.mma, accumulators in TMEM), written for B200 (sm_100a).
//
//   y[m,n] = sum_k x[m,k] * (scale[n,k/64] * code[n,k] + bias[n,k/64]),   m < M <= 32
//
// With a handful of activation rows the matvec is still a pure weight stream (0.5625 B per
// weight); what a SIMT or mma.sync kernel runs out of is issue slots, because every extra
// activation row costs instructions in the inner loop. Here the rows cost nothing: the 128
// weight rows of a tile are the M dimension of the MMA, the (up to 32) activation rows its N
// dimension, so one tcgen05.mma of shape 128 x 32 x 16 serves all of them and the SM's lanes only
// expand codes. It is affine_qmm with the operand roles swapped and a streaming schedule:
//
//   warp 4        producer: one tiled TMA load per stage brings the packed codes of a 128-row tile,
//                 KC k-blocks (of 64 codes) wide, as a 128 x 128-byte box with the 128-byte swizzle
//                 (conflict-free 16-byte reads; per-row bulk copies of 128 bytes were measured
//                 nine times slower - the copy engine's request rate, not its bandwidth), plus
//                 the tiled loads of the activation k-blocks (32 x 64 bf16) of the stage.
//   warps 6-13    dequantisers: two threads per weight row read 16 packed bytes from the stage,
//                 expand to bf16 (w = bf16(scale*q + bias): one rounding, the contract of
//                 affine_qmm) and write the row slice with tcgen05.st into a ring of A operands
//                 in TENSOR MEMORY (TMEM lane = weight row). Shared memory then carries only the
//                 packed codes and the activations: a dequantised A tile in shared memory would be
//                 written and read back at 16 KB per k-block each, three quarters of the SM's
//                 shared-memory bandwidth at the rate HBM delivers codes. Scales and biases come
//                 straight from global memory, loaded a stage ahead.
//   warp 5        MMA issuer: 4 x tcgen05.mma (M=128, N=32, K=16; A from TMEM, B from shared
//                 memory) per k-block into one of two TMEM accumulators; tcgen05.commit hands A
//                 slots, stages and finished accumulators back.
//   warps 0-3     epilogue: tcgen05.ld the accumulator of the previous tile (TMEM lane = weight
//                 row, column = activation row) while the next tile streams, and store y so that
//                 consecutive lanes write consecutive n.
//
// CTAs are persistent over (row tile, K slice) work items; matrices with fewer row tiles than
// SMs are cut along K and leave f32 partial sums that a small kernel adds in slice order
// (deterministic). The GeGLU form streams a gate and an up tile per stage into two accumulators
// and multiplies in the epilogue. Every mbarrier wait is bounded; on a time-out the kernel
// records it in the device status word, frees its TMEM and returns.
#include "common.cuh"
#include "qmv.hpp"

#include <cuda.h>

#include <algorithm>
#include <mutex>

namespace lthn {

constexpr int TC_ROWS = 128;   // weight rows per tile (MMA M)
constexpr int TC_NB = 32;      // activation rows per MMA (MMA N)
constexpr int TC_KC = 4;       // k-blocks per stage
constexpr int TC_PTILE = TC_ROWS * TC_KC * 32;  // packed codes of one stage and set: 128 rows x 128 bytes
constexpr int TC_DQ_THREADS = 256;
constexpr int TC_THREADS = 6 * 32 + TC_DQ_THREADS;  // 4 epilogue warps, producer, issuer, 8 dequant warps
constexpr int TC_XTILE = TC_NB * 128;     // one activation k-block in shared memory, bytes
constexpr int TC_ASLOTS = 3;              // ring of dequantised A operands in TMEM, 128 columns each

template <int SETS>
struct TcSmem {
    static constexpr int STAGES = SETS == 2 ? 4 : 5;
    static constexpr int WSLOTS = TC_ASLOTS;
    static constexpr int PACKED = SETS * TC_PTILE;
    static constexpr int X_OFF = PACKED;
    // scales and biases of the stage: per set and row 8 bytes of each (4 k-blocks), then padding
    static constexpr int SB_OFF = X_OFF + TC_KC * TC_XTILE;
    static constexpr int STAGE_BYTES = SB_OFF + 4096;  // a multiple of 1024
    static constexpr int BAR_OFF = STAGES * STAGE_BYTES;
    static constexpr int TOTAL = BAR_OFF + 512 + 1024 /*alignment slack*/;
    static_assert(SETS * TC_ROWS * 16 <= 4096, "scale/bias area");
    // An A slot holds GR k-blocks of every set (128 columns): the issuer and the dequantisers shake
    // hands once per slot, not once per k-block - with 64 cycles of tensor work per k-block the
    // per-k-block handshake (wait, fence, commit in one issuing thread) was what bounded the
    // first version at 730 cycles per k-block with the arithmetic and the loads switched off.
    static constexpr int GR = SETS == 2 ? 2 : 4;
    static constexpr int SLOT_COLS = SETS * GR * 32;
    // TMEM columns: two accumulator buffers of SETS*32, then the A ring
    static constexpr int A_COL0 = 2 * SETS * TC_NB;
    static constexpr int TMEM_COLS = 512;
    static_assert(A_COL0 + WSLOTS * SLOT_COLS <= TMEM_COLS, "TMEM budget");
};

struct TcArgs {
    const uint32_t* wq[2];
    const uint16_t* scales[2];
    const uint16_t* biases[2];
    void* y;          // [M, N] f32 or bf16 (ks == 1)
    float* part;      // ks > 1: [ks][SETS][M][N] f32 partial sums
    uint32_t* status;
    int M, N, K;
    int ntiles, ks;   // row tiles, K slices per tile
    int y_dtype;
};

// ---- tcgen05 / TMA wrappers (cta_group::1, no multicast) --------------------------------------
__device__ __forceinline__ void tc_tmem_alloc(uint32_t* smem_dst, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_dst)), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_tmem_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tc_tmem_dealloc(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
// D[tmem] (+)= A[tmem] * B[smem descriptor]
__device__ __forceinline__ void tc_umma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
// 16 consecutive 32-bit columns of this thread's TMEM lane
__device__ __forceinline__ void tc_tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
          "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]) : "memory");
}
__device__ __forceinline__ void tc_tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tc_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tc_tma_load_2d(void* dst, const CUtensorMap* map, int c0, int c1, uint64_t* bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 ::"r"(smem_u32(dst)), "l"(map), "r"(c0), "r"(c1), "r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tc_tma_load_3d(void* dst, const CUtensorMap* map, int c0, int c1, int c2, uint64_t* bar) {
    asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
                 ::"r"(smem_u32(dst)), "l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tc_cp_async8(void* dst, const void* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(smem_u32(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void tc_cp_async4(void* dst, const void* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(smem_u32(dst)), "l"(src) : "memory");
}
// the mbarrier receives one (pre-counted) arrival when every cp.async this thread has issued so far has landed
__device__ __forceinline__ void tc_cp_async_arrive(uint64_t* bar) {
    asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tc_tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
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
__device__ __forceinline__ void tc_tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Bounded wait on an mbarrier phase. try_wait parks the thread until the phase completes or a
// hardware time limit passes, so a waiting warp does not take issue slots from the working ones.
// The bound is wall time (about 50 ms on the global timer): a wait that runs out makes the role
// record its status bit and leave, the other roles then run out in turn, and the kernel ends
// within a fraction of a second whatever went wrong.
__device__ __forceinline__ bool tc_wait(uint64_t* bar, uint32_t parity) {
    uint32_t done = 0;
    uint64_t t0 = 0;
    for (uint32_t it = 0;; ++it) {
        asm volatile("{\n\t.reg .pred p;\n\t"
                     "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
                     "selp.u32 %0, 1, 0, p;\n\t}"
                     : "=r"(done) : "r"(smem_u32(bar)), "r"(parity) : "memory");
        if (done) return true;
        if ((it & 63) == 63) {
            uint64_t now;
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
            if (t0 == 0) t0 = now;
            else if (now - t0 > 50000000ull) return false;
        }
    }
}

// K-major operand, 128-byte swizzle, 8-row groups 1024 bytes apart (tile base 1024-aligned)
__device__ __forceinline__ uint64_t tc_desc(uint32_t smem_addr) {
    return (uint64_t)((smem_addr & 0x3FFFFu) >> 4) | ((uint64_t)1 << 16) | ((uint64_t)(1024 >> 4) << 32) |
           ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
}

__device__ __forceinline__ uint32_t tc_bf16x2_sub(uint32_t a, uint32_t b) {
    uint32_t d;
    asm("sub.rn.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
    return d;
}
__device__ __forceinline__ uint32_t tc_bf16x2_fma(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t d;
    asm("fma.rn.bf16x2 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}
// 8 codes of one packed word -> 8 bf16 weights in memory order (one 16-byte chunk):
// (w>>4i & 0x000F000F) | 0x43004300 is the bf16 pair {128+q, 128+q'}; subtracting 128 is exact and
// the fused multiply-add rounds scale*q + bias once.
__device__ __forceinline__ uint4 tc_dequant_word(uint32_t w, uint32_t s2, uint32_t b2) {
    const uint32_t k128 = 0x43004300u;
    uint32_t p0 = (w & 0x000F000Fu) | k128;
    uint32_t p1 = ((w >> 4) & 0x000F000Fu) | k128;
    uint32_t p2 = ((w >> 8) & 0x000F000Fu) | k128;
    uint32_t p3 = ((w >> 12) & 0x000F000Fu) | k128;
    p0 = tc_bf16x2_fma(tc_bf16x2_sub(p0, k128), s2, b2);
    p1 = tc_bf16x2_fma(tc_bf16x2_sub(p1, k128), s2, b2);
    p2 = tc_bf16x2_fma(tc_bf16x2_sub(p2, k128), s2, b2);
    p3 = tc_bf16x2_fma(tc_bf16x2_sub(p3, k128), s2, b2);
    uint4 o;
    o.x = __byte_perm(p0, p1, 0x5410);
    o.y = __byte_perm(p2, p3, 0x5410);
    o.z = __byte_perm(p0, p1, 0x7632);
    o.w = __byte_perm(p2, p3, 0x7632);
    return o;
}

__device__ __forceinline__ float tc_gelu_tanh(float x) {
    // gelu_tanh as hipGemma4Q4HostGELU (engine/hip/hip_gemma4_q4_layer.go:3582-3597)
    const float k0 = 0.7978845608028654f, k1 = 0.044715f;
    return 0.5f * x * (1.0f + tanhf(k0 * (x + k1 * x * x * x)));
}

// k-blocks [kb0, kb1) of K slice `slice` out of `ks`: whole stages of TC_KC k-blocks (slices may
// differ by one stage), so every stage starts at a multiple of TC_KC
__device__ __forceinline__ void tc_slice_range(int KB, int ks, int slice, int& kb0, int& kb1) {
    const int nst = (KB + TC_KC - 1) / TC_KC;
    kb0 = (int)((int64_t)nst * slice / ks) * TC_KC;
    kb1 = min(KB, (int)((int64_t)nst * (slice + 1) / ks) * TC_KC);
}

template <int SETS>
__global__ void __launch_bounds__(TC_THREADS, 1) qmv_tc_kernel(const __grid_constant__ CUtensorMap x_map, const __grid_constant__ CUtensorMap w_map0,
              const __grid_constant__ CUtensorMap w_map1, const TcArgs a) {
    using S = TcSmem<SETS>;
    constexpr int STAGES = S::STAGES, WSLOTS = S::WSLOTS;
    constexpr int ACC_COLS = SETS * TC_NB;      // TMEM columns of one accumulator buffer
    constexpr int TMEM_COLS = S::TMEM_COLS;
    extern __shared__ unsigned char tc_smem_raw[];
    unsigned char* smem = (unsigned char*)(((uintptr_t)tc_smem_raw + 1023) & ~(uintptr_t)1023);
    uint64_t* bars = (uint64_t*)(smem + S::BAR_OFF);
    uint64_t* full = bars;                         // [STAGES] producer -> dequantisers + issuer
    uint64_t* empty = full + STAGES;               // [STAGES] 8 dequant warps + 1 commit
    uint64_t* wfull = empty + STAGES;              // [WSLOTS] 8 dequant warps (all sets of the k-block written)
    uint64_t* wempty = wfull + WSLOTS;             // [WSLOTS] 1 commit
    uint64_t* afull = wempty + WSLOTS;             // [2] 1 commit
    uint64_t* aempty = afull + 2;                  // [2] 4 epilogue warps
    uint32_t* tmem_slot = (uint32_t*)(aempty + 2);

    pdl_trigger();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int KB = a.K >> 6;
    const int items = a.ntiles * a.ks;

    if (threadIdx.x == 0) {
        // full: the producer's expect_tx arrival + one cp.async completion arrival per producer lane
        for (int s = 0; s < STAGES; s++) { mbar_init(&full[s], 33); mbar_init(&empty[s], 9); }  // empty: 8 dequant warps + the issuer's commit
        for (int s = 0; s < WSLOTS; s++) { mbar_init(&wfull[s], 8); mbar_init(&wempty[s], 1); }
        for (int s = 0; s < 2; s++) { mbar_init(&afull[s], 1); mbar_init(&aempty[s], 4); }
        mbar_fence_init();
    }
    if (warp == 5) {
        tc_tmem_alloc(tmem_slot, TMEM_COLS);
        tc_tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    bool ok = true;

    if (warp == 4) {
        // ---- producer: packed weights never depend on the previous kernel; the activations do ----
        int sit = 0;  // stage uses so far
        bool waited = false;
        for (int item = blockIdx.x; item < items && ok; item += gridDim.x) {
            const int rt = item / a.ks, slice = item - rt * a.ks;
            const int64_t n0 = (int64_t)rt * TC_ROWS;
            int kb0, kb1;
            tc_slice_range(KB, a.ks, slice, kb0, kb1);
            for (int kb = kb0; kb < kb1 && ok; kb += TC_KC, sit++) {
                const int st = sit % STAGES, kc = min(TC_KC, kb1 - kb);
                ok = tc_wait(&empty[st], ((sit / STAGES) & 1) ^ 1);
                if (!ok) atomicOr(a.status, 1u << 16);  // which wait ran out
                if (!ok) break;
                unsigned char* sb = smem + (size_t)st * S::STAGE_BYTES;
                if (lane == 0) {
                    // the boxes are always whole (k-blocks past K and rows past N or M arrive as zeros)
                    mbar_expect_tx(&full[st], (uint32_t)(SETS * TC_PTILE + TC_KC * TC_XTILE));
                    tc_tma_load_2d(sb, &w_map0, kb * 8, (int)n0, &full[st]);
                    if (SETS == 2) tc_tma_load_2d(sb + TC_PTILE, &w_map1, kb * 8, (int)n0, &full[st]);
                }
                if (!waited) { pdl_wait(); waited = true; }
                // Scales and biases of the stage's four k-blocks: 8 bytes per row and tensor, fetched by
                // this warp's lanes with cp.async (4 rows per lane) into the stage, so they travel
                // with the same depth of prefetch as the codes and no dequantiser ever waits on a
                // global load. 8-byte copies where the row pitch keeps them aligned (K a multiple
                // of 256), two 4-byte copies for K a multiple of 128, plain 2-byte loads otherwise.
#pragma unroll
                for (int set = 0; set < SETS; set++)
#pragma unroll
                    for (int i = 0; i < TC_ROWS / 32; i++) {
                        const int r = lane + 32 * i;
                        const int64_t e = min(n0 + r, (int64_t)a.N - 1) * KB + kb;
                        unsigned char* d = sb + S::SB_OFF + (size_t)(set * TC_ROWS + r) * 16;
                        if ((KB & 3) == 0) {
                            tc_cp_async8(d, a.scales[set] + e);
                            tc_cp_async8(d + 8, a.biases[set] + e);
                        } else if ((KB & 1) == 0) {
                            tc_cp_async4(d, a.scales[set] + e);
                            tc_cp_async4(d + 8, a.biases[set] + e);
                            if (kc > 2) { tc_cp_async4(d + 4, a.scales[set] + e + 2); tc_cp_async4(d + 12, a.biases[set] + e + 2); }
                        } else {
                            for (int j = 0; j < kc; j++) {
                                ((uint16_t*)d)[j] = __ldg(a.scales[set] + e + j);
                                ((uint16_t*)d)[4 + j] = __ldg(a.biases[set] + e + j);
                            }
                        }
                    }
                if ((KB & 1) == 0) tc_cp_async_arrive(&full[st]);
                else tc_arrive(&full[st]);  // plain stores above: an ordinary (releasing) arrival
                // the stage's four activation k-blocks in one load: x viewed as [k-block][row][64]
                if (lane == 0) tc_tma_load_3d(sb + S::X_OFF, &x_map, 0, 0, kb, &full[st]);
            }
        }
        if (!ok && lane == 0) atomicOr(a.status, 512u);
    } else if (warp == 5) {
        // ---- MMA issuer ------------------------------------------------------------------------
        if (lane == 0) {
            // c f32, a/b bf16, K-major both, N = 32, M = 128
            const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(TC_NB >> 3) << 17) | ((128u >> 4) << 24);
            int sit = 0, wit = 0, ait = 0;
            for (int item = blockIdx.x; item < items && ok; item += gridDim.x, ait++) {
                const int rt = item / a.ks, slice = item - rt * a.ks;
                int kb0, kb1;
                tc_slice_range(KB, a.ks, slice, kb0, kb1);
                const int acc = ait & 1;
                ok = tc_wait(&aempty[acc], ((ait >> 1) & 1) ^ 1);  // the epilogue has drained this buffer
                if (!ok) atomicOr(a.status, 2u << 16);  // which wait ran out
                if (!ok) break;
                tc_fence_after();
                const uint32_t d0 = tmem_base + acc * ACC_COLS;
                for (int kb = kb0; kb < kb1 && ok; kb += TC_KC, sit++) {
                    const int st = sit % STAGES, kc = min(TC_KC, kb1 - kb);
                    // no wait on full[st] here: the dequantisers arrive on wfull only after they have seen
                    // full[st] complete, which also covers the activation tiles of the stage
                    const uint64_t bd0 = tc_desc(smem_u32(smem + (size_t)st * S::STAGE_BYTES + S::X_OFF));
                    for (int g0 = 0; g0 < kc && ok; g0 += S::GR, wit++) {
                        const int ws = wit % WSLOTS;
                        ok = tc_wait(&wfull[ws], (wit / WSLOTS) & 1);
                        if (!ok) atomicOr(a.status, 4u << 16);  // which wait ran out
                        if (!ok) break;
                        tc_fence_after();
                        const uint32_t slot = tmem_base + S::A_COL0 + ws * S::SLOT_COLS;
#pragma unroll
                        for (int jj = 0; jj < S::GR; jj++) {
                            if (g0 + jj < kc) {
#pragma unroll
                                for (int set = 0; set < SETS; set++)
#pragma unroll
                                    for (int q = 0; q < 4; q++)
                                        // A: 128 lanes x 8 columns (16 bf16) per MMA; B: the activation k-block, 32 bytes per K=16 step
                                        tc_umma_ts(d0 + set * TC_NB, slot + (jj * SETS + set) * 32 + q * 8,
                                                   bd0 + (uint64_t)((g0 + jj) * (TC_XTILE >> 4) + q * 2), idesc,
                                                   (kb + g0 + jj > kb0 || q > 0) ? 1u : 0u);
                            }
                        }
                        tc_commit(&wempty[ws]);
                    }
                    if (ok) tc_commit(&empty[st]);
                }
                if (ok) tc_commit(&afull[acc]);
            }
            if (!ok) atomicOr(a.status, 1024u);
        }
    } else if (warp >= 6) {
        // ---- dequantisers ------------------------------------------------------------------------
        // A warp may touch the TMEM lanes of its quadrant (warp % 4): its 32 lanes take the 32 weight
        // rows of that quadrant, and the two warps of a quadrant take one half of the k-block each.
        // The 8 lanes of a quarter-warp hit 8 different 16-byte columns of the swizzled stage.
        // A warp may touch the TMEM lanes of its quadrant (warp % 4): its 32 lanes take the 32 weight
        // rows of that quadrant, and the two warps of a quadrant take one half of every k-block each.
        // Every warp works on every group, in order: a warp that skipped groups could get two phases
        // ahead of an A slot's barrier, which a parity wait cannot tell from "free". The 8 lanes of a
        // quarter-warp hit 8 different 16-byte columns of the swizzled stage.
        const int quad = warp & 3, part = (warp - 6) >> 2;
        const int row = quad * 32 + lane;
        int sit = 0, wit = 0;
        for (int item = blockIdx.x; item < items && ok; item += gridDim.x) {
            const int slice = item % a.ks;
            int kb0, kb1;
            tc_slice_range(KB, a.ks, slice, kb0, kb1);
            for (int kb = kb0; kb < kb1 && ok; kb += TC_KC, sit++) {
                const int st = sit % STAGES, kc = min(TC_KC, kb1 - kb);
                ok = tc_wait(&full[st], (sit / STAGES) & 1);
                if (!ok) atomicOr(a.status, 8u << 16);  // which wait ran out
                if (!ok) break;
                const unsigned char* sb = smem + (size_t)st * S::STAGE_BYTES;
                // this row's scales (low half) and biases (high half) of the stage's four k-blocks
                uint32_t sbc[SETS][TC_KC];
#pragma unroll
                for (int set = 0; set < SETS; set++) {
                    const uint4 v = *(const uint4*)(sb + S::SB_OFF + (size_t)(set * TC_ROWS + row) * 16);
                    sbc[set][0] = (v.x & 0xffffu) | (v.z << 16);
                    sbc[set][1] = (v.x >> 16) | (v.z & 0xffff0000u);
                    sbc[set][2] = (v.y & 0xffffu) | (v.w << 16);
                    sbc[set][3] = (v.y >> 16) | (v.w & 0xffff0000u);
                }
                static_assert(TC_KC == 4, "four k-blocks of scales per 8 bytes");
                for (int g0 = 0; g0 < kc && ok; g0 += S::GR, wit++) {
                    const int ws = wit % WSLOTS;
                    ok = tc_wait(&wempty[ws], ((wit / WSLOTS) & 1) ^ 1);
                    if (!ok) atomicOr(a.status, 16u << 16);  // which wait ran out
                    if (!ok) break;
                    tc_fence_after();
                    const uint32_t slot = tmem_base + ((uint32_t)(quad * 32) << 16) + S::A_COL0 + ws * S::SLOT_COLS;
#pragma unroll
                    for (int jj = 0; jj < S::GR; jj++) {
                        const int j = g0 + jj;
                        if (j < kc) {
#pragma unroll
                            for (int set = 0; set < SETS; set++) {
                                const uint32_t sbv = sbc[set][j];
                                const uint32_t s2 = (sbv & 0xffffu) | (sbv << 16);
                                const uint32_t b2 = (sbv >> 16) | (sbv & 0xffff0000u);
                                {
                                    const uint4 pk = *(const uint4*)(sb + (size_t)set * TC_PTILE + row * 128 + (((j * 2 + part) ^ (row & 7)) << 4));
                                    const uint32_t w4[4] = {pk.x, pk.y, pk.z, pk.w};
                                    uint32_t cells[16];  // 32 bf16 weights: cell c holds k = 2c (low half) and 2c+1
#pragma unroll
                                    for (int i = 0; i < 4; i++) {
                                        const uint4 o = tc_dequant_word(w4[i], s2, b2);
                                        cells[4 * i] = o.x; cells[4 * i + 1] = o.y; cells[4 * i + 2] = o.z; cells[4 * i + 3] = o.w;
                                    }
                                    tc_tmem_st16(slot + (jj * SETS + set) * 32 + part * 16, cells);
                                }
                            }
                        }
                    }
                    tc_tmem_st_wait();
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) tc_arrive(&wfull[ws]);
                }
                // this warp has read everything it needs from the stage
                __syncwarp();
                if (lane == 0) tc_arrive(&empty[st]);
            }
        }
        if (!ok && lane == 0) atomicOr(a.status, 2048u);
    } else {
        // ---- epilogue: warp w reads TMEM lanes 32w..32w+31 (weight rows) -----------------------------
        int ait = 0;
        for (int item = blockIdx.x; item < items && ok; item += gridDim.x, ait++) {
            const int rt = item / a.ks, slice = item - rt * a.ks;
            const int acc = ait & 1;
            ok = tc_wait(&afull[acc], (ait >> 1) & 1);
            if (!ok) atomicOr(a.status, 32u << 16);  // which wait ran out
            if (!ok) break;
            tc_fence_after();
            const uint32_t taddr = tmem_base + ((uint32_t)(warp * 32) << 16) + acc * ACC_COLS;
            uint32_t r[32];
            tc_tmem_ld32(taddr, r);
            float v[32];
            if (SETS == 2) {
                uint32_t u[32];
                tc_tmem_ld32(taddr + TC_NB, u);
                tc_tmem_ld_wait();
                if (a.ks == 1) {
#pragma unroll
                    for (int m = 0; m < 32; m++) v[m] = tc_gelu_tanh(__uint_as_float(r[m])) * __uint_as_float(u[m]);
                } else {
                    // partial sums of both sets: the summing kernel applies the GeGLU
                    const int64_t n = (int64_t)rt * TC_ROWS + warp * 32 + lane;
                    if (n < a.N) {
                        float* p0 = a.part + ((int64_t)(slice * 2 + 0) * a.M) * a.N + n;
                        float* p1 = a.part + ((int64_t)(slice * 2 + 1) * a.M) * a.N + n;
#pragma unroll
                        for (int m = 0; m < 32; m++)
                            if (m < a.M) { p0[(int64_t)m * a.N] = __uint_as_float(r[m]); p1[(int64_t)m * a.N] = __uint_as_float(u[m]); }
                    }
                }
            } else {
                tc_tmem_ld_wait();
#pragma unroll
                for (int m = 0; m < 32; m++) v[m] = __uint_as_float(r[m]);
            }
            // the values are in registers: the issuer may reuse this accumulator
            tc_fence_before();
            __syncwarp();
            if (lane == 0) tc_arrive(&aempty[acc]);
            if (SETS == 2 && a.ks > 1) continue;
            const int64_t n = (int64_t)rt * TC_ROWS + warp * 32 + lane;
            if (n >= a.N) continue;
            if (a.ks > 1) {
                float* p = a.part + ((int64_t)slice * a.M) * a.N + n;
#pragma unroll
                for (int m = 0; m < 32; m++) if (m < a.M) p[(int64_t)m * a.N] = v[m];
            } else if (a.y_dtype == LTHN_DTYPE_BF16) {
                uint16_t* p = (uint16_t*)a.y + n;
#pragma unroll
                for (int m = 0; m < 32; m++) if (m < a.M) p[(int64_t)m * a.N] = f32_to_bf16_bits(v[m]);
            } else {
                float* p = (float*)a.y + n;
#pragma unroll
                for (int m = 0; m < 32; m++) if (m < a.M) p[(int64_t)m * a.N] = v[m];
            }
        }
        if (!ok && lane == 0) atomicOr(a.status, 4096u);
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 5) tc_tmem_dealloc(tmem_base, TMEM_COLS);
}

// y = sum over slices (in order) of the partial sums; with two sets the GeGLU of the two sums
__global__ void qmv_tc_sum_kernel(const float* __restrict__ part, int ks, int sets, int64_t n, void* __restrict__ y, int y_dtype) {
    pdl_trigger();
    pdl_wait();
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    float v = 0.f, u = 0.f;
    for (int s = 0; s < ks; s++) {
        v += part[((int64_t)s * sets) * n + i];
        if (sets == 2) u += part[((int64_t)s * sets + 1) * n + i];
    }
    if (sets == 2) v = tc_gelu_tanh(v) * u;
    if (y_dtype == LTHN_DTYPE_BF16) ((uint16_t*)y)[i] = f32_to_bf16_bits(v);
    else ((float*)y)[i] = v;
}

// ---- host side --------------------------------------------------------------------------------
typedef CUresult (*TcEncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                    const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                    CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static TcEncodeTiledFn tc_encode_fn() {
    static std::mutex mu;
    static TcEncodeTiledFn fn = nullptr;
    std::lock_guard<std::mutex> lk(mu);
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
            fn = (TcEncodeTiledFn)p;
    }
    return fn;
}

bool qmv_tc_available(const QmvCall& c) {
    if (c.M < 1 || c.M > TC_NB || c.K % 64 != 0 || c.K < 64 || c.N < 1) return false;
    if (c.N >= ((int64_t)1 << 31) || c.K >= ((int64_t)1 << 31)) return false;
    bool aligned = (((uintptr_t)c.wq) & 15) == 0 && (((uintptr_t)c.scales | (uintptr_t)c.biases) & 7) == 0;
    if (c.wq2) aligned = aligned && (((uintptr_t)c.wq2) & 15) == 0 && (((uintptr_t)c.scales2 | (uintptr_t)c.biases2) & 7) == 0;
    return aligned && tc_encode_fn() != nullptr;
}

template <int SETS>
static int32_t tc_launch_t(cudaStream_t st, const CUtensorMap& map, const CUtensorMap& w0, const CUtensorMap& w1, const TcArgs& a, int grid) {
    static int attr_dev = -1;
    static std::mutex mu;
    int dev = 0;
    LTHN_CUDA_TRY(cudaGetDevice(&dev));
    {
        std::lock_guard<std::mutex> lk(mu);
        if (attr_dev != dev) {
            LTHN_CUDA_TRY(cudaFuncSetAttribute(qmv_tc_kernel<SETS>, cudaFuncAttributeMaxDynamicSharedMemorySize, TcSmem<SETS>::TOTAL));
            attr_dev = dev;
        }
    }
    LTHN_CUDA_TRY(launch_k(qmv_tc_kernel<SETS>, dim3(grid), dim3(TC_THREADS), (size_t)TcSmem<SETS>::TOTAL, st, map, w0, w1, a));
    return LTHN_OK;
}

// x_bf16: bf16 activations, row m at x_bf16 + m*x_ld (16-byte aligned rows). Serves c.M <= 32; see qmv_tc_available.
int32_t qmv_tc_launch(cudaStream_t st, const QmvCall& c, const uint16_t* x_bf16, int64_t x_ld) {
    static_assert(TcSmem<1>::TOTAL <= 227 * 1024 && TcSmem<2>::TOTAL <= 227 * 1024, "shared memory budget");
    if (((uintptr_t)x_bf16 & 15) != 0 || (x_ld * 2) % 16 != 0) return fail(LTHN_ERR_INVALID, "affine_qmv: bf16 activation rows must be 16-byte aligned");
    CUtensorMap map;
    // x [M, K] viewed as [k-block][row][64]: a box of 4 k-blocks x 32 rows lands as four K-major
    // operand tiles (rows past M and k-blocks past K are zero-filled)
    const cuuint64_t dims[3] = {64, (cuuint64_t)c.M, (cuuint64_t)(c.K / 64)};
    const cuuint64_t strides[2] = {(cuuint64_t)x_ld * 2, 128};
    const cuuint32_t box[3] = {64, TC_NB, TC_KC};
    const cuuint32_t estr[3] = {1, 1, 1};
    CUresult cr = tc_encode_fn()(&map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, (void*)x_bf16, dims, strides, box, estr,
                                 CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                                 CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (cr != CUDA_SUCCESS) return fail(LTHN_ERR_CUDA, "affine_qmv: cuTensorMapEncodeTiled failed (" + std::to_string((int)cr) + ")");
    // packed codes as a [N][K/8] matrix of 32-bit words: a stage is a box of 128 rows x 32 words
    CUtensorMap wmap[2];
    for (int set = 0; set < (c.wq2 ? 2 : 1); set++) {
        const cuuint64_t wdims[2] = {(cuuint64_t)(c.K / 8), (cuuint64_t)c.N};
        const cuuint64_t wstrides[1] = {(cuuint64_t)c.K / 2};
        const cuuint32_t wbox[2] = {TC_KC * 8, TC_ROWS};
        cr = tc_encode_fn()(&wmap[set], CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, (void*)(set ? c.wq2 : c.wq), wdims, wstrides, wbox, estr,
                            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (cr != CUDA_SUCCESS) return fail(LTHN_ERR_CUDA, "affine_qmv: cuTensorMapEncodeTiled (weights) failed (" + std::to_string((int)cr) + ")");
    }
    if (!c.wq2) wmap[1] = wmap[0];
    int dev = 0, sms = 148;
    LTHN_CUDA_TRY(cudaGetDevice(&dev));
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const int sets = c.wq2 ? 2 : 1;
    const int KB = (int)(c.K / 64);
    TcArgs a{};
    a.wq[0] = c.wq; a.scales[0] = c.scales; a.biases[0] = c.biases;
    a.wq[1] = c.wq2; a.scales[1] = c.scales2; a.biases[1] = c.biases2;
    a.y = c.y; a.M = c.M; a.N = (int)c.N; a.K = (int)c.K; a.y_dtype = c.y_dtype;
    a.ntiles = (int)((c.N + TC_ROWS - 1) / TC_ROWS);
    // fewer row tiles than SMs: cut K so that every SM streams (slices of at least 4 k-blocks)
    a.ks = 1;
    if (a.ntiles < sms) a.ks = std::max(1, std::min(std::min(sms / a.ntiles, (KB + TC_KC - 1) / TC_KC), 16));
    a.status = device_status_word();
    if (!a.status) return fail(LTHN_ERR_CUDA, "affine_qmv: no device status word");
    if (a.ks > 1) {
        void* ws = nullptr;
        int32_t rc = scratch_get((size_t)a.ks * sets * c.M * c.N * sizeof(float), &ws, 4);
        if (rc) return rc;
        a.part = (float*)ws;
    }
    const int grid = std::min(a.ntiles * a.ks, sms);
    int32_t rc = sets == 2 ? tc_launch_t<2>(st, map, wmap[0], wmap[1], a, grid) : tc_launch_t<1>(st, map, wmap[0], wmap[1], a, grid);
    if (rc) return rc;
    if (a.ks > 1) {
        const int64_t n = (int64_t)c.M * c.N;
        LTHN_CUDA_TRY(launch_k(qmv_tc_sum_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, st, (const float*)a.part, a.ks, sets, n,
                               c.y, c.y_dtype));
    }
    return LTHN_OK;
}

}  // namespace lthn
