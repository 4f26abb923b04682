// decode_persistent.cu — every decoder block of one token in ONE kernel (batch 1, one GPU), sm_100a.
//
// Why. A batch-1 decode step of a Gemma-style block is five small kernels' worth of work
// (q|k|v matvec, head norms + RoPE + attention, o matvec, gate|up GeGLU matvec, down matvec), each
// of which moves only a few MB of 4-bit weights. Launched one by one (even inside a CUDA graph,
// even with programmatic dependent launch) every kernel pays its own ramp: the weight stream
// stops at each boundary and restarts from a cold pipeline. Here one cooperative grid of one CTA
// per SM walks all blocks; phases are separated by grid-wide barriers, and the weight stream is
// decoupled from them:
//
//  * warps 8 and 9 of every CTA are producers. They know the CTA's whole work list for the token (weights
//    do not depend on activations) and keep a ring of shared-memory slots full with 1-D bulk
//    (TMA) copies of 16-row x <=44-group weight pieces plus cp.async copies of their scales and
//    biases, running ahead of the consumers across phase boundaries and grid barriers. While the
//    grid is synchronising and the next phase's activations are being prepared, the weights of
//    that phase are already landing.
//  * warps 0..7 are consumers. Per phase they turn the activation vector into the three int8
//    digit planes of the integer tensor-core matvec (x = sx*(d0 + d1/128 + d2/16384), exact
//    integer dot products, f32 per-group scaling; the arithmetic of qmv_i8_kernel.cuh) in
//    shared memory, then multiply ring slots with mma.sync.m16n8k32.u8.s8 and add the eight
//    warps' partial sums in a fixed order. The residual RMSNorm pairs are part of the activation
//    preparation (every CTA computes them redundantly from L2; CTA 0 stores the residual stream).
//  * attention runs as two 128-thread groups per CTA over (kv head, key chunk) items: the head
//    norms, RoPE and the KV append of the new token are folded into the items, and the last item
//    of a kv head to finish merges that head's chunk partials (a counter per kv head), so the
//    phase needs no barrier of its own.
//
// Every wait (ring slot, grid barrier) is bounded in time. A wait that runs out sets a bit in the
// device status word and an abort flag; from then on every wait returns at once, the CTAs fall
// through the remaining control flow without touching data, the producer waits (bounded) for its
// copies in flight, and the kernel returns by itself. The host reports LTHN_ERR_DEVICE_WAIT.
//
// The reference decodes a token through per-op kernels chained by its engine
// (engine/metal/decode_step.go, engine/hip/hip_gemma4_q4_forward.go); this kernel replaces that
// chain for one row on one GPU and leaves the same buffers behind (the last down-projection
// output and the residual stream), so the lm_head with its fused final norm follows unchanged.
#include "attn_item.cuh"
#include "common.cuh"
#include "decoder_kernels.hpp"

#include <algorithm>
#include <mutex>

namespace lthn {

constexpr int PK_CW = 8;                  // consumer warps
constexpr int PK_CT = PK_CW * 32;         // consumer threads
constexpr int PK_THREADS = PK_CT + 64;    // plus the two producer warps
constexpr int PK_RS_MAX = 1440;           // bytes between weight rows of a slot (44 groups * 32 B + pad)
constexpr int PK_SB_OFF = 16 * PK_RS_MAX; // scales of a slot
constexpr int PK_SB_HALF = 16 * PERSIST_SLOT_G * 2;             // biases follow the scales
constexpr int PK_SLOT_BYTES = PK_SB_OFF + 2 * PK_SB_HALF;       // 25856
constexpr int PK_MAX_SLOTS = 8;
constexpr int PK_PART_OFF = 1024;         // [2][PK_CW][16] f32 partial sums
constexpr int PK_DIG_OFF = 2048;          // activation digits (per phase), attention scratch
constexpr uint64_t PK_WAIT_NS = 50ull * 1000 * 1000;

// status bits of this kernel (device status word)
constexpr uint32_t PK_ST_SLOT_EMPTY = 1u << 13, PK_ST_SLOT_FULL = 1u << 14, PK_ST_GRID = 1u << 15;

// shared-memory row stride of a slot holding ks groups per row: 8 words mod 32, so the 8-byte
// fragment loads of a half-warp (8 rows x 4 pieces) fall into 32 different banks
__host__ __device__ inline int pk_row_stride(int ks) { return ks * 32 + ((32 - ks * 32) & 127); }

__device__ __forceinline__ void pk_mma(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void pk_mma_z(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
                 : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0));
}
__device__ __forceinline__ void pk_cp_async8(void* dst, const void* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(smem_u32(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void pk_cp_async4(void* dst, const void* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(smem_u32(dst)), "l"(src) : "memory");
}
// one (pre-counted) arrival on the mbarrier once every cp.async this thread has issued has landed
__device__ __forceinline__ void pk_cp_async_arrive(uint64_t* bar) {
    asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void pk_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ uint64_t pk_now() {
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ void pk_bar_consumers() { asm volatile("bar.sync 1, %0;" ::"n"(PK_CT) : "memory"); }
__device__ __forceinline__ void pk_bar_group(int g) { asm volatile("bar.sync %0, 128;" ::"r"(2 + g) : "memory"); }
__device__ __forceinline__ float pk_gelu(float x) {
    const float k0 = 0.7978845608028654f, k1 = 0.044715f;
    return 0.5f * x * (1.0f + tanhf(k0 * (x + k1 * x * x * x)));
}

// Bounded mbarrier wait. `abort` is the CTA's abort word in shared memory: once set, nothing waits.
__device__ __forceinline__ bool pk_wait(uint64_t* bar, uint32_t parity, volatile uint32_t* abort, const PersistArgs& a, uint32_t bit) {
    if (*abort) return false;
    uint32_t done = 0;
    uint64_t t0 = 0;
    for (uint32_t it = 0;; ++it) {
        asm volatile("{\n\t.reg .pred p;\n\t"
                     "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
                     "selp.u32 %0, 1, 0, p;\n\t}"
                     : "=r"(done) : "r"(smem_u32(bar)), "r"(parity) : "memory");
        if (done) return true;
        if ((it & 63) == 63) {
            if (*abort) return false;
            const uint64_t now = pk_now();
            if (t0 == 0) t0 = now;
            else if (now - t0 > PK_WAIT_NS) break;
        }
    }
    *abort = 1u;
    atomicExch(a.sync + 2, 1u);
    atomicOr(a.status, bit);
    return false;
}

// Grid-wide barrier of the consumer warps of every CTA (the producers never join: they touch only
// weights), split into arrive and wait so that loads which do not depend on the other CTAs can be
// issued in between. sync[0] counts arrivals and grows for the life of the launch (the waiters poll
// the counter itself: the last arrival is visible to them one L2 access after it lands); sync[2]
// is the abort flag.
__device__ __forceinline__ void pk_grid_arrive(const PersistArgs& a, volatile uint32_t* abort) {
    pk_bar_consumers();
    // the barrier above ordered the CTA's writes before this thread; the release makes them visible with the count
    if (threadIdx.x == 0 && !*abort) asm volatile("red.release.gpu.global.add.u32 [%0], %1;" ::"l"(a.sync), "r"(1u) : "memory");
}
__device__ __noinline__ bool pk_grid_wait(const PersistArgs& a, uint32_t& epoch, volatile uint32_t* abort, volatile uint32_t* okflag) {
    if (threadIdx.x == 0) {
        uint32_t ok = 0;
        if (!*abort) {
            const uint32_t target = (epoch + 1u) * gridDim.x;
            const uint64_t t0 = pk_now();
            for (uint32_t it = 0;; ++it) {
                uint32_t v;
                asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(a.sync) : "memory");
                if (v >= target) { ok = 1; break; }
                if ((it & 31) == 31) {
                    uint32_t ab;
                    asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(ab) : "l"(a.sync + 2) : "memory");
                    if (ab) break;
                    if (pk_now() - t0 > PK_WAIT_NS) { atomicOr(a.status, PK_ST_GRID); break; }
                }
            }
            if (!ok) { *abort = 1u; atomicExch(a.sync + 2, 1u); }
        }
        *okflag = ok;
    }
    epoch++;
    pk_bar_consumers();
    return *okflag != 0;
}

// f64 sum over the consumer threads (sh: 8 doubles)
__device__ __forceinline__ double pk_block_sum(double v, double* sh, int lane, int warp) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    pk_bar_consumers();
    if (lane == 0) sh[warp] = v;
    pk_bar_consumers();
    double t = 0.0;
#pragma unroll
    for (int w = 0; w < PK_CW; w++) t += sh[w];
    return t;
}

// Digit planes of U groups at once (independent dependency chains interleave). x[u][q]: elements
// 2*lane+q of group u. dg: 192 bytes per group - three planes of 64 digit bytes in MMA fragment
// order; gc: (sx, sx-weighted sum of the group's activations) per group.
template <int U>
__device__ __forceinline__ void pk_digitise(const float (&x)[U][2], const bool (&live)[U], int lane, unsigned char* const (&dg)[U], float2* const (&gc)[U]) {
    float amax[U];
#pragma unroll
    for (int u = 0; u < U; u++)  // non-negative floats order like their bit patterns
        amax[u] = __uint_as_float(__reduce_max_sync(0xffffffffu, __float_as_uint(fmaxf(fabsf(x[u][0]), fabsf(x[u][1])))));
    int isum[U];
    float sxv[U];
#pragma unroll
    for (int u = 0; u < U; u++) {
        const float sx = amax[u] * (1.0f / 127.0f);
        const float inv = amax[u] > 0.f ? __fdividef(127.0f, amax[u]) : 0.f;
        const float sx1 = sx * (1.0f / 128.0f);
        sxv[u] = sx;
        isum[u] = 0;
#pragma unroll
        for (int q = 0; q < 2; q++) {
            const float x0 = x[u][q];
            const float d0 = rintf(x0 * inv);
            const float r1 = fmaf(-d0, sx, x0);
            const float d1 = rintf(r1 * inv * 128.0f);
            const float r2 = fmaf(-d1, sx1, r1);
            const float d2 = rintf(r2 * inv * 16384.0f);
            const int i0 = (int)d0, i1 = (int)d1, i2 = (int)d2;
            isum[u] += i0 * 16384 + i1 * 128 + i2;
            // element e of the group: word e>>3 of the row piece, nibble e&7. Thread t of a fragment
            // owns words 2t (first MMA) and 2t+1 (second); even nibbles feed the low k half, odd
            // nibbles the high k half.
            const int e = 2 * lane + q;
            const int off = ((((e >> 3) & 1) * 4 + (e >> 4)) * 2 + (e & 1)) * 4 + ((e & 7) >> 1);
            if (live[u]) {
                dg[u][off] = (unsigned char)(i0 & 0xff);
                dg[u][64 + off] = (unsigned char)(i1 & 0xff);
                dg[u][128 + off] = (unsigned char)(i2 & 0xff);
            }
        }
    }
#pragma unroll
    for (int u = 0; u < U; u++) isum[u] = __reduce_add_sync(0xffffffffu, isum[u]);
#pragma unroll
    for (int u = 0; u < U; u++)
        if (live[u] && lane == 0) *gc[u] = make_float2(sxv[u], (float)isum[u] * (sxv[u] * (1.0f / 16384.0f)));
}

struct PkSmem {
    uint64_t* full;
    uint64_t* empty;
    double* nsum;
    volatile uint32_t* abort;
    volatile uint32_t* okflag;
    float* part;
    unsigned char* dig;
    unsigned char* ring;
};

// Activation vector of a matvec phase -> digit planes. src: G*64 f32 values; `scale_w` (optional):
// per-element weights applied after dividing by rms (the trailing RMSNorm of a residual pair).
__device__ __noinline__ void pk_prepare_digits(const PkSmem& sm, const float* src, bool src_smem, int G, float rms, const float* w_next, int lane,
                                                  int warp) {
    constexpr int U = 4;
    float2* gcb = (float2*)(sm.dig + (size_t)G * 192);
    for (int g0 = warp; g0 < G; g0 += PK_CW * U) {
        float x[U][2];
        bool live[U];
        unsigned char* dg[U];
        float2* gc[U];
#pragma unroll
        for (int u = 0; u < U; u++) {
            const int g = g0 + u * PK_CW;
            live[u] = g < G;
            const int gg = live[u] ? g : g0;
            const int e = gg * 64 + 2 * lane;
            float2 v = src_smem ? *(const float2*)(src + e) : __ldcg((const float2*)(src + e));
            x[u][0] = v.x; x[u][1] = v.y;
            dg[u] = sm.dig + (size_t)gg * 192;
            gc[u] = gcb + gg;
        }
        pk_digitise<U>(x, live, lane, dg, gc);
    }
    pk_bar_consumers();
}

// Static weights of a residual RMSNorm pair, fetched before the grid barrier in front of it is
// waited for. Thread (warp, lane) owns elements 2*lane, 2*lane+1 of the groups warp, warp+8, ...
constexpr int PK_NV = 11;  // groups per thread: hidden <= 64 * 8 * 11 = 5632
struct PkNormW {
    float2 wp[PK_NV], wn[PK_NV];
};
__device__ __noinline__ void pk_norm_prefetch(PkNormW& nw, const float* w_post, const float* w_next, int G, int lane, int warp) {
#pragma unroll
    for (int i = 0; i < PK_NV; i++) {
        const int g = warp + i * PK_CW;
        const int e = g * 64 + 2 * lane;
        nw.wp[i] = (w_post && g < G) ? __ldg((const float2*)(w_post + e)) : make_float2(0.f, 0.f);
        nw.wn[i] = g < G ? __ldg((const float2*)(w_next + e)) : make_float2(0.f, 0.f);
    }
}

// Residual RMSNorm pair in front of a matvec (every CTA computes it; CTA 0 stores the stream):
//   h_out = h_in + rmsnorm(avec) * w_post   (skipped when avec == nullptr: h_out is h_in)
//   x     = rmsnorm(h_out) * w_next  -> digit planes in shared memory
// Thread (warp, lane) owns elements 2*lane, 2*lane+1 of the groups warp, warp+8, ...: everything
// stays in registers (one memory round trip for avec and h_in), every step is branch-free so the
// groups' arithmetic interleaves, and the sums of squares run on four f64 accumulators.
__device__ __noinline__ void pk_norm_prologue(const PkSmem& sm, const PersistArgs& a, const float* avec, const float* h_in, float* h_out,
                                              const PkNormW& nw, int lane, int warp) {
    const int H = a.H, G = H >> 6;
    const double inv_h = a.inv_h;
    float2 av[PK_NV], hv[PK_NV];
#pragma unroll
    for (int i = 0; i < PK_NV; i++) {
        const int g = warp + i * PK_CW;
        const int e = g * 64 + 2 * lane;
        hv[i] = g < G ? __ldcg((const float2*)(h_in + e)) : make_float2(0.f, 0.f);
        av[i] = (avec && g < G) ? __ldcg((const float2*)(avec + e)) : make_float2(0.f, 0.f);
    }
    if (avec) {
        double s4[4] = {0.0, 0.0, 0.0, 0.0};
#pragma unroll
        for (int i = 0; i < PK_NV; i++) {  // zeros beyond the vector
            s4[(2 * i) & 3] += (double)__fmul_rn(av[i].x, av[i].x);
            s4[(2 * i + 1) & 3] += (double)__fmul_rn(av[i].y, av[i].y);
        }
        const double ss = pk_block_sum((s4[0] + s4[1]) + (s4[2] + s4[3]), sm.nsum, lane, warp);
        const FastDiv k = fast_div_by(fast_rms(ss, inv_h, a.eps));
#pragma unroll
        for (int i = 0; i < PK_NV; i++) {
            hv[i].x = __fadd_rn(hv[i].x, __fmul_rn(fast_div(av[i].x, k), nw.wp[i].x));
            hv[i].y = __fadd_rn(hv[i].y, __fmul_rn(fast_div(av[i].y, k), nw.wp[i].y));
        }
        if (blockIdx.x == 0) {
#pragma unroll
            for (int i = 0; i < PK_NV; i++) {
                const int g = warp + i * PK_CW;
                if (g < G) *(float2*)(h_out + g * 64 + 2 * lane) = hv[i];
            }
        }
    }
    double s4[4] = {0.0, 0.0, 0.0, 0.0};
#pragma unroll
    for (int i = 0; i < PK_NV; i++) {
        s4[(2 * i) & 3] += (double)__fmul_rn(hv[i].x, hv[i].x);
        s4[(2 * i + 1) & 3] += (double)__fmul_rn(hv[i].y, hv[i].y);
    }
    const double ss2 = pk_block_sum((s4[0] + s4[1]) + (s4[2] + s4[3]), sm.nsum, lane, warp);
    const FastDiv k2 = fast_div_by(fast_rms(ss2, inv_h, a.eps));
    // the normed vector goes through shared memory: one rolled copy of the digit conversion serves every phase
    float* xs = (float*)(sm.dig + (((size_t)G * 200 + 15) & ~(size_t)15));
#pragma unroll
    for (int i = 0; i < PK_NV; i++) {
        const int g = warp + i * PK_CW;
        if (g < G)
            *(float2*)(xs + g * 64 + 2 * lane) = make_float2(__fmul_rn(fast_div(hv[i].x, k2), nw.wn[i].x), __fmul_rn(fast_div(hv[i].y, k2), nw.wn[i].y));
    }
    __syncwarp();  // a warp converts the groups it wrote
    pk_prepare_digits(sm, xs, true, G, 1.f, nullptr, lane, warp);
}

// Digit planes that another phase left in global memory (G groups: G*192 digit bytes, then G
// (sx, sum) pairs) -> shared memory. Every load is issued before the first store.
__device__ __noinline__ void pk_digits_from_global(const PkSmem& sm, const unsigned char* src, int G) {
    const int n16 = (G * 200) >> 4;
    const uint4* s4 = (const uint4*)src;
    uint4* d4 = (uint4*)sm.dig;
    for (int i0 = threadIdx.x; i0 < n16; i0 += 8 * PK_CT) {
        uint4 v[8];
#pragma unroll
        for (int k = 0; k < 8; k++) {
            const int i = i0 + k * PK_CT;
            v[k] = i < n16 ? __ldcg(s4 + i) : make_uint4(0u, 0u, 0u, 0u);
        }
#pragma unroll
        for (int k = 0; k < 8; k++) {
            const int i = i0 + k * PK_CT;
            if (i < n16) d4[i] = v[k];
        }
    }
    pk_bar_consumers();
}

// This CTA's share of a vector in global memory -> digit planes in global memory (groups cta,
// cta + grid, ...; one warp per group).
__device__ __noinline__ void pk_digitise_share(const float* src, unsigned char* dst, int G, int lane, int warp) {
    float2* gcb = (float2*)(dst + (size_t)G * 192);
    for (int g = blockIdx.x + warp * gridDim.x; g < G; g += PK_CW * gridDim.x) {
        const float2 v = __ldcg((const float2*)(src + (size_t)g * 64 + 2 * lane));
        const float x[1][2] = {{v.x, v.y}};
        const bool live[1] = {true};
        unsigned char* const dg[1] = {dst + (size_t)g * 192};
        float2* const gc[1] = {gcb + g};
        pk_digitise<1>(x, live, lane, dg, gc);
    }
}

// One matvec phase of the consumers: this CTA's row blocks (b = cta, cta+grid, ...), each of
// ph.nsl ring slots. FUSE: rows 0-7 of a slot are gate rows, rows 8-15 the same rows of up;
// out[row] = gelu_tanh(gate) * up. it_base: the ring position at entry (the caller advances it by pk_blocks() * nsl).
// 
__device__ __forceinline__ uint32_t pk_blocks(const PersistPhase& ph) {
    return (int)blockIdx.x < ph.nblk ? (uint32_t)((ph.nblk - 1 - (int)blockIdx.x) / (int)gridDim.x + 1) : 0u;
}
__device__ __noinline__ void pk_matvec(uint64_t* full, uint64_t* empty, volatile uint32_t* abort, float* part, const unsigned char* dig,
                                       const unsigned char* ring, const PersistArgs& a, PersistPhase ph, bool fuse, float* out, int nslots,
                                       uint32_t it_base) {
    // The eight consumer warps split into T teams that work on different row blocks at the same time, so
    // that the latency of one ring slot (wait, fragment loads, MMAs, hand-back) overlaps with the others':
    // T = 4 teams of two warps when the CTA has at least four row blocks in this phase, 2 x 4 or 1 x 8 below.
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nrb = (int)pk_blocks(ph);
    const int tshift = nrb >= 4 ? 2 : nrb >= 2 ? 1 : 0;
    const int T = 1 << tshift, WT = PK_CW >> tshift;
    const int team = warp / WT, wt = warp - team * WT;
    const int gq = lane >> 2, t = lane & 3;
    const float2* gcb = (const float2*)(dig + (size_t)ph.G * 192);
    constexpr uint32_t NIB = 0x0F0F0F0Fu;
    const bool colrow = t < 2;  // columns of activation row 0 (the only row)
    const float planew = !colrow ? 0.f : (t & 1) ? (1.0f / 2097152.0f) : (1.0f / 128.0f);
    int jj = 0;
    for (int j = team; j < nrb; j += T, jj++) {
        const int b = blockIdx.x + j * gridDim.x;
        float acc0 = 0.f, acc1 = 0.f, accb = 0.f;
        // ring order: (wave of T row blocks, slice, team), so that the slots in flight always serve every team
        const int wave = j >> tshift, inwave = min(T, nrb - (wave << tshift));
        for (int sl = 0; sl < ph.nsl; sl++) {
            const uint32_t it = it_base + (uint32_t)((wave << tshift) * ph.nsl + sl * inwave + team);
            const uint32_t lap = it / (uint32_t)nslots;
            const int slot = (int)(it - lap * (uint32_t)nslots);
            const bool ok = __all_sync(0xffffffffu, pk_wait(&full[slot], lap & 1, abort, a, PK_ST_SLOT_FULL));
            const int g0 = sl * ph.KS, ks = min(ph.KS, ph.G - g0), RS = pk_row_stride(ks);
            const unsigned char* sb = ring + (size_t)slot * PK_SLOT_BYTES;
            if (ok) {
                const uint16_t* sp = (const uint16_t*)(sb + PK_SB_OFF) + gq * ks;
                const uint16_t* bp = (const uint16_t*)(sb + PK_SB_OFF + PK_SB_HALF) + (gq + 8 * (t & 1)) * ks;
                const unsigned char* rowp = sb + (size_t)gq * RS + t * 8;
                const unsigned char* dgp = dig + (size_t)g0 * 192 + (gq < 3 ? gq : 0) * 64 + t * 8;
                // Six groups of the team's share (g = wt, wt+WT, ...) are in flight together: twelve independent
                // MMAs whose loads and unpacking overlap. No branches: a group past the end of the slot repeats the
                // warp's first group with weight zero.
                constexpr int U = 6;
                for (int gb = wt; gb < ks; gb += U * WT) {
                    uint2 wa[U], wb[U], b0[U], b1[U];
                    float gx[U], gy[U], s0[U], s1[U], bb[U];
#pragma unroll
                    for (int u = 0; u < U; u++) {
                        const int g = gb + u * WT;
                        const bool live = g < ks;
                        const int gg = live ? g : wt;
                        b0[u] = *(const uint2*)(dgp + gg * 192);
                        b1[u] = *(const uint2*)(dgp + gg * 192 + 32);
                        if (gq >= 3) { b0[u] = make_uint2(0u, 0u); b1[u] = b0[u]; }
                        wa[u] = *(const uint2*)(rowp + gg * 32);
                        wb[u] = *(const uint2*)(rowp + (size_t)8 * RS + gg * 32);
                        const float2 gc = gcb[g0 + gg];
                        gx[u] = live ? gc.x * planew : 0.f;
                        gy[u] = (live && colrow) ? gc.y : 0.f;
                        s0[u] = bf16_bits_to_f32(sp[gg]);
                        s1[u] = bf16_bits_to_f32(sp[8 * ks + gg]);
                        bb[u] = bf16_bits_to_f32(bp[gg]);
                    }
                    float f0[U], f1[U];
#pragma unroll
                    for (int u = 0; u < U; u++) {
                        int c0[4], c1[4];
                        pk_mma_z(c0, wa[u].x & NIB, wb[u].x & NIB, (wa[u].x >> 4) & NIB, (wb[u].x >> 4) & NIB, b0[u].x, b0[u].y);
                        pk_mma_z(c1, wa[u].y & NIB, wb[u].y & NIB, (wa[u].y >> 4) & NIB, (wb[u].y >> 4) & NIB, b1[u].x, b1[u].y);
                        f0[u] = (float)((c0[0] + c1[0]) * 128 + (c0[1] + c1[1])) * gx[u];
                        f1[u] = (float)((c0[2] + c1[2]) * 128 + (c0[3] + c1[3])) * gx[u];
                    }
#pragma unroll
                    for (int u = 0; u < U; u++) {
                        acc0 = fmaf(s0[u], f0[u], acc0);
                        acc1 = fmaf(s1[u], f1[u], acc1);
                        accb = fmaf(bb[u], gy[u], accb);
                    }
                }
            }
            __syncwarp();
            // this warp is done with the slot: the team's WT warps bring the PK_CW arrivals the barrier expects
            if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(&empty[slot])), "r"(T) : "memory");
        }
        // lanes t and t^1 hold the two plane halves of the same outputs; even t finishes row gq,
        // odd t row gq+8 (each also carries that row's bias term)
        const bool odd = t & 1;
        const float send = odd ? acc0 : acc1;
        const float recv = __shfl_xor_sync(0xffffffffu, send, 1);
        const float res = (odd ? acc1 : acc0) + recv + accb;
        float* p0 = part + (size_t)((team * 2 + (jj & 1)) * WT) * 16;  // [T][2][WT][16]
        if (colrow) p0[wt * 16 + gq + 8 * (t & 1)] = res;
        asm volatile("bar.sync %0, %1;" ::"r"(4 + team), "r"(WT * 32) : "memory");
        if (wt == jj % WT) {
            if (!fuse) {
                if (lane < 16) {
                    float v = 0.f;
                    for (int w = 0; w < WT; w++) v += p0[w * 16 + lane];
                    out[(size_t)b * 16 + lane] = v;
                }
            } else if (lane < 8) {
                float g = 0.f, u = 0.f;
                for (int w = 0; w < WT; w++) { g += p0[w * 16 + lane]; u += p0[w * 16 + 8 + lane]; }
                out[(size_t)b * 8 + lane] = pk_gelu(g) * u;
            }
        }
    }
}

// ---- attention: (kv head, key chunk) items on the CTA's two 128-thread groups (attn_item.cuh) ------
// the finished output of the item's heads (s.q[h][d], reused as a staging area) -> digit planes of the o
// projection's input in global memory; one warp per group of 64
template <int D, int GQ>
__device__ __forceinline__ void pk_att_emit(const PersistArgs& a, AttnItemSmem<D, GQ>& s, int qh0, int lane, int warp) {
    constexpr int GH = D / 64;  // groups per head
    const int Gq = (a.Hq * D) >> 6;
    float2* gcb = (float2*)(a.dig_att + (size_t)Gq * 192);
#pragma unroll 1
    for (int gi = warp; gi < GQ * GH; gi += 4) {
        const int h = gi / GH, j = gi - h * GH;
        const float2 v = *(const float2*)(&s.q[h][j * 64 + 2 * lane]);
        const float x[1][2] = {{v.x, v.y}};
        const bool live[1] = {true};
        const int g = (qh0 + h) * GH + j;
        unsigned char* const dg[1] = {a.dig_att + (size_t)g * 192};
        float2* const gc[1] = {gcb + g};
        pk_digitise<1>(x, live, lane, dg, gc);
    }
}

template <int D, int GQ>
__device__ __noinline__ void pk_attention_item(const PersistArgs& a, const PersistLayer& L, AttnItemSmem<D, GQ>& s, int grp, int kvh, int chunk,
                                               int used, int pos, int64_t lane_off) {
    AttnItemArgs it;
    it.qkv = a.qkv; it.n_q = L.n_q; it.n_k = L.n_k; it.rope = a.rope;
    it.kc = L.kcache + lane_off; it.vc = L.vcache + lane_off;
    it.part = a.part; it.counter = a.sync + 64;
    it.Hq = a.Hq; it.Hkv = a.Hkv; it.nchunks_cap = a.nchunks_cap; it.max_len = a.max_len;
    it.eps = a.eps; it.scale = a.attn_scale;
    const int lane = threadIdx.x & 31, warp = (threadIdx.x & 127) >> 5;
    attn_item<D, GQ>(it, s, [grp] { pk_bar_group(grp); },
                     [&](AttnItemSmem<D, GQ>& sm, int qh0) { pk_att_emit<D, GQ>(a, sm, qh0, lane, warp); }, kvh, chunk, used, pos);
}

template <int D, int GQ>
__global__ void __launch_bounds__(PK_THREADS, 1) decode_persistent_kernel(const __grid_constant__ PersistArgs a) {
    extern __shared__ __align__(128) unsigned char psm[];
    PkSmem sm;
    sm.full = (uint64_t*)psm;
    sm.empty = sm.full + PK_MAX_SLOTS;
    sm.nsum = (double*)(psm + 128);
    sm.abort = (volatile uint32_t*)(psm + 192);
    sm.okflag = (volatile uint32_t*)(psm + 196);
    sm.part = (float*)(psm + PK_PART_OFF);
    sm.dig = psm + PK_DIG_OFF;
    sm.ring = psm + a.ring_off;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int nslots = a.nslots;
    if (tid == 0) {
        for (int i = 0; i < nslots; i++) { mbar_init(&sm.full[i], 33); mbar_init(&sm.empty[i], PK_CW); }
        mbar_fence_init();
        *sm.abort = 0u;
        *sm.okflag = 0u;
    }
    __syncthreads();

    if (warp >= PK_CW) {
        // ---- producers: the whole token's weight pieces of this CTA, in the consumers' order. Warp 8
        // issues the bulk copies of the 16 row pieces of a slot, warp 9 the cp.async copies of their
        // scales and biases; both wait for the slot to be free and neither waits for the other.
        const bool rows_warp = warp == PK_CW;
        uint32_t it = 0;
        bool ok = true;
        for (int li = 0; li < a.nlayers && ok; li++) {
            const PersistLayer& L = a.layers[li];
            for (int p = 0; p < 4 && ok; p++) {
                const PersistPhase ph = a.ph[p];
                const bool fuse = p == 2;
                const uint32_t* w0 = p == 0 ? L.qkv_w : p == 1 ? L.o_w : p == 2 ? L.gate_w : L.down_w;
                const uint16_t* s0 = p == 0 ? L.qkv_s : p == 1 ? L.o_s : p == 2 ? L.gate_s : L.down_s;
                const uint16_t* b0 = p == 0 ? L.qkv_b : p == 1 ? L.o_b : p == 2 ? L.gate_b : L.down_b;
                const uint32_t* w1 = fuse ? L.up_w : w0;
                const uint16_t* s1 = fuse ? L.up_s : s0;
                const uint16_t* b1 = fuse ? L.up_b : b0;
                const int64_t rowbytes = (int64_t)ph.G * 32;
                // the consumers' order: (wave of T row blocks, slice, team) - see pk_matvec
                const int nrb = (int)pk_blocks(ph);
                const int tshift = nrb >= 4 ? 2 : nrb >= 2 ? 1 : 0;
                for (int wave = 0; (wave << tshift) < nrb && ok; wave++) {
                    const int inwave = min(1 << tshift, nrb - (wave << tshift));
                    for (int sl = 0; sl < ph.nsl && ok; sl++) {
                      for (int k = 0; k < inwave; k++, it++) {
                        const int b = blockIdx.x + ((wave << tshift) + k) * gridDim.x;
                        const int slot = it % nslots;
                        ok = __all_sync(0xffffffffu, pk_wait(&sm.empty[slot], ((it / nslots) & 1) ^ 1, sm.abort, a, PK_ST_SLOT_EMPTY));
                        if (!ok) break;
                        const int g0 = sl * ph.KS, ks = min(ph.KS, ph.G - g0), RS = pk_row_stride(ks);
                        unsigned char* sb = sm.ring + (size_t)slot * PK_SLOT_BYTES;
                        if (rows_warp) {
                            if (lane == 0) mbar_expect_tx(&sm.full[slot], (uint32_t)(16 * ks * 32));
                            __syncwarp();
                            if (lane < 16) {
                                const bool second = fuse && lane >= 8;
                                const int64_t grow = fuse ? (int64_t)b * 8 + (lane & 7) : (int64_t)b * 16 + lane;
                                const unsigned char* src = (const unsigned char*)(second ? w1 : w0) + grow * rowbytes + (int64_t)g0 * 32;
                                bulk_g2s(sb + (size_t)lane * RS, src, (uint32_t)(ks * 32), &sm.full[slot]);
                            }
                        } else {
                            // Lane l copies for row l & 15 the units l >> 4, (l >> 4) + 2, ... of the row's scales and
                            // biases: units of 8 bytes (4 groups) where the piece allows it, of 4 bytes otherwise.
                            // Nothing but additions per unit - this warp sets the pace of the ring.
                            const bool wide = ((ks | g0 | ph.G) & 3) == 0;
                            const int ug = wide ? 4 : 2, upr = ks / ug;
                            const int r = lane & 15;
                            const bool second = fuse && r >= 8;
                            const int64_t grow = fuse ? (int64_t)b * 8 + (r & 7) : (int64_t)b * 16 + r;
                            const uint16_t* ps = (second ? s1 : s0) + grow * ph.G + g0;
                            const uint16_t* pb = (second ? b1 : b0) + grow * ph.G + g0;
                            unsigned char* d = sb + PK_SB_OFF + (size_t)r * ks * 2;
                            if (wide) {
#pragma unroll 6
                                for (int u = lane >> 4; u < upr; u += 2) {
                                    pk_cp_async8(d + u * 8, ps + u * 4);
                                    pk_cp_async8(d + PK_SB_HALF + u * 8, pb + u * 4);
                                }
                            } else {
#pragma unroll 4
                                for (int u = lane >> 4; u < upr; u += 2) {
                                    pk_cp_async4(d + u * 4, ps + u * 2);
                                    pk_cp_async4(d + PK_SB_HALF + u * 4, pb + u * 2);
                                }
                            }
                            pk_cp_async_arrive(&sm.full[slot]);
                        }
                      }
                    }
                }
            }
        }
        if (!ok) {
            // gave up: let the copies already issued land before the CTA's shared memory goes away
            const uint32_t first = it > (uint32_t)nslots ? it - nslots : 0u;
            for (uint32_t j = first; j < it; j++) {
                uint32_t done = 0;
                const uint64_t t0 = pk_now();
                while (!done && pk_now() - t0 < PK_WAIT_NS) {
                    asm volatile("{\n\t.reg .pred p;\n\t"
                                 "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
                                 "selp.u32 %0, 1, 0, p;\n\t}"
                                 : "=r"(done) : "r"(smem_u32(&sm.full[j % nslots])), "r"((j / nslots) & 1) : "memory");
                }
            }
        }
        return;
    }

    // ---- consumers --------------------------------------------------------------------------------
    using Att = AttnItemSmem<D, GQ>;
    Att* att_s = (Att*)sm.dig;  // two of them; the digits are dead during the attention phase
    uint32_t it = 0, epoch = 0;
    const float* hcur = a.h0;
    float* halt = a.h1;
    const int pos = a.row_pos[0];
    const int64_t lane_off = (int64_t)a.row_lane[0] * a.lane_stride;
    constexpr int CH = 16 * (512 / D > 0 ? 512 / D : 1);
    const int used = min(a.nchunks_cap, (pos + CH) / CH);
    const int Gh = a.H >> 6, Gq = (a.Hq * D) >> 6, Gf = a.F >> 6;
    PkNormW nw;
    pk_norm_prefetch(nw, nullptr, a.layers[0].n_input, Gh, lane, warp);
    for (int li = 0; li < a.nlayers; li++) {
        const PersistLayer& L = a.layers[li];
        // q|k|v: the previous block's post-FFN norm and residual add (none for the first block), this block's input norm
        pk_norm_prologue(sm, a, li ? a.a : nullptr, hcur, halt, nw, lane, warp);
        if (li) { const float* t = hcur; hcur = halt; halt = (float*)t; }
        pk_matvec(sm.full, sm.empty, sm.abort, sm.part, sm.dig, sm.ring, a, a.ph[0], false, a.qkv, nslots, it);
        it += pk_blocks(a.ph[0]) * a.ph[0].nsl;
        pk_grid_arrive(a, sm.abort);
        const bool live = pk_grid_wait(a, epoch, sm.abort, sm.okflag);
        // attention (the barrier's verdict is the same for every thread of the CTA); leaves the digit
        // planes of its output in global memory
        if (live) {
            const int grp = warp >> 2;
            const int nitems = a.Hkv * used;
            for (int i = blockIdx.x * 2 + grp; i < nitems; i += gridDim.x * 2)
                pk_attention_item<D, GQ>(a, L, att_s[grp], grp, i % a.Hkv, i / a.Hkv, used, pos, lane_off);
        }
        pk_grid_arrive(a, sm.abort);
        pk_norm_prefetch(nw, L.n_post_attn, L.n_pre_ff, Gh, lane, warp);  // for the gate|up phase, while the grid gathers
        pk_grid_wait(a, epoch, sm.abort, sm.okflag);
        // o
        pk_digits_from_global(sm, a.dig_att, Gq);
        pk_matvec(sm.full, sm.empty, sm.abort, sm.part, sm.dig, sm.ring, a, a.ph[1], false, a.a, nslots, it);
        it += pk_blocks(a.ph[1]) * a.ph[1].nsl;
        pk_grid_arrive(a, sm.abort);
        pk_grid_wait(a, epoch, sm.abort, sm.okflag);
        // gate | up: post-attention norm + residual add, pre-FFN norm
        {
            pk_norm_prologue(sm, a, a.a, hcur, halt, nw, lane, warp);
            const float* t = hcur; hcur = halt; halt = (float*)t;
        }
        pk_matvec(sm.full, sm.empty, sm.abort, sm.part, sm.dig, sm.ring, a, a.ph[2], true, a.act, nslots, it);
        it += pk_blocks(a.ph[2]) * a.ph[2].nsl;
        pk_grid_arrive(a, sm.abort);
        pk_grid_wait(a, epoch, sm.abort, sm.okflag);
        // the GeGLU vector -> digit planes: every CTA converts its share, then all of them read the whole
        pk_digitise_share(a.act, a.dig_act, Gf, lane, warp);
        pk_grid_arrive(a, sm.abort);
        if (li + 1 < a.nlayers) pk_norm_prefetch(nw, L.n_post_ff, a.layers[li + 1].n_input, Gh, lane, warp);
        pk_grid_wait(a, epoch, sm.abort, sm.okflag);
        // down
        pk_digits_from_global(sm, a.dig_act, Gf);
        pk_matvec(sm.full, sm.empty, sm.abort, sm.part, sm.dig, sm.ring, a, a.ph[3], false, a.a, nslots, it);
        it += pk_blocks(a.ph[3]) * a.ph[3].nsl;
        if (li + 1 < a.nlayers) {
            pk_grid_arrive(a, sm.abort);
            pk_grid_wait(a, epoch, sm.abort, sm.okflag);
        }
    }
}

// ---- host ---------------------------------------------------------------------------------------
static PersistPhase pk_phase(int64_t N, int64_t K, bool fuse) {
    PersistPhase p{};
    p.G = (int)(K >> 6);
    p.nsl = (p.G + PERSIST_SLOT_G - 1) / PERSIST_SLOT_G;
    // slices of a multiple of four groups where the row allows it: their scales move as 8-byte copies
    const int unit = (p.G & 3) == 0 ? 4 : 2;
    p.KS = ((p.G + p.nsl - 1) / p.nsl + unit - 1) / unit * unit;
    p.nsl = (p.G + p.KS - 1) / p.KS;
    p.nblk = (int)(fuse ? N / 8 : N / 16);
    return p;
}

template <int D>
static size_t pk_att_bytes() { return 2 * sizeof(AttnItemSmem<D, 2>); }

bool persist_supported(int H, int Hq, int Hkv, int D, int F, std::string* why) {
    auto no = [&](const char* m) { if (why) *why = m; return false; };
    if (D != 64 && D != 128 && D != 256) return no("head_dim must be 64, 128 or 256");
    if (Hq != 2 * Hkv) return no("two query heads per kv head");
    if (Hkv > 32) return no("at most 32 kv heads");
    const int64_t Kq = (int64_t)Hq * D, Nqkv = (int64_t)(Hq + 2 * Hkv) * D;
    if (H % 128 || Kq % 128 || F % 128) return no("hidden, q width and ffn must be multiples of 128");
    if (H % 16 || Nqkv % 16 || F % 8) return no("row counts must be multiples of 16");
    if (H > 64 * PK_CW * PK_NV) return no("hidden wider than 5632");
    return true;
}

size_t persist_digit_bytes(int Hq, int D, int F) { return (size_t)std::max(Hq * D, F) / 64 * 200; }

int32_t persist_plan(int H, int Hq, int Hkv, int D, int F, PersistArgs* a, size_t* smem) {
    std::string why;
    if (!persist_supported(H, Hq, Hkv, D, F, &why)) return fail(LTHN_ERR_INVALID, "persistent decode: " + why);
    const int64_t Kq = (int64_t)Hq * D, Nqkv = (int64_t)(Hq + 2 * Hkv) * D;
    a->ph[0] = pk_phase(Nqkv, H, false);
    a->ph[1] = pk_phase(H, Kq, false);
    a->ph[2] = pk_phase(F, H, true);
    a->ph[3] = pk_phase(H, F, false);
    const int Gmax = std::max({H >> 6, (int)(Kq >> 6), F >> 6});
    size_t dig = (size_t)Gmax * 200;
    dig = std::max(dig, (((size_t)(H >> 6) * 200 + 15) & ~(size_t)15) + (size_t)H * 4);  // a norm phase also stages the normed vector
    dig = std::max(dig, D == 64 ? pk_att_bytes<64>() : D == 128 ? pk_att_bytes<128>() : pk_att_bytes<256>());
    dig = (dig + 127) & ~(size_t)127;
    a->ring_off = (int)(PK_DIG_OFF + dig);
    const size_t budget = 227 * 1024;
    if ((size_t)a->ring_off + 2 * (size_t)PK_SLOT_BYTES > budget) return fail(LTHN_ERR_INVALID, "persistent decode: the activation digits leave no room for the weight ring");
    a->nslots = (int)std::min<size_t>(PK_MAX_SLOTS, (budget - a->ring_off) / PK_SLOT_BYTES);
    *smem = (size_t)a->ring_off + (size_t)a->nslots * PK_SLOT_BYTES;
    return LTHN_OK;
}

template <int D>
static int32_t pk_launch(cudaStream_t s, const PersistArgs& a, size_t smem) {
    static std::mutex mu;
    static int attr_dev = -1, grid_cache = 0;
    int dev = 0;
    LTHN_CUDA_TRY(cudaGetDevice(&dev));
    auto kern = decode_persistent_kernel<D, 2>;
    int grid;
    {
        std::lock_guard<std::mutex> lk(mu);
        if (attr_dev != dev) {
            LTHN_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
            int sms = 0, occ = 0, coop = 0;
            LTHN_CUDA_TRY(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
            LTHN_CUDA_TRY(cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, dev));
            LTHN_CUDA_TRY(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, kern, PK_THREADS, smem));
            if (!coop || occ < 1) return fail(LTHN_ERR_CUDA, "persistent decode: the kernel cannot be launched cooperatively on this device");
            grid_cache = sms;
            attr_dev = dev;
        }
        grid = grid_cache;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid); cfg.blockDim = dim3(PK_THREADS); cfg.dynamicSmemBytes = smem; cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeCooperative;
    attr[0].val.cooperative = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    LTHN_CUDA_TRY(cudaLaunchKernelEx(&cfg, kern, a));
    return LTHN_OK;
}

// the sync words are cleared on the same stream before every launch
int32_t launch_decode_persistent(cudaStream_t s, const PersistArgs& a, size_t smem) {
    LTHN_CUDA_TRY(cudaMemsetAsync(a.sync, 0, PERSIST_SYNC_WORDS * sizeof(uint32_t), s));
    if (a.D == 64) return pk_launch<64>(s, a, smem);
    if (a.D == 128) return pk_launch<128>(s, a, smem);
    if (a.D == 256) return pk_launch<256>(s, a, smem);
    return fail(LTHN_ERR_INVALID, "persistent decode: unsupported head_dim");
}

}  // namespace lthn
