// qmv_i8_kernel.cuh — affine_qmv for one or two activation rows on the integer tensor-core path
// (mma.sync m16n8k32, u8 x s8 -> s32), written for B200 (sm_100a).
//
// Why this shape of kernel. At batch 1 the matvec is a stream of 4-bit codes from HBM; what
// limits it on the SM is the number of instructions spent per weight byte. One m16n8k32
// multiplies 16 rows x 32 codes (256 weight bytes) by 8 columns and B200 retires one per
// 2.5 SM cycles (measured: 105 G/s over 148 SMs, the same rate as the bf16 m16n8k16), four
// times the rate the HBM stream needs, while unpacking eight codes to bytes costs three
// logic ops. The activations are converted once per CTA to block fixed point exactly as in
// the dp4a kernel: for each group g of 64 consecutive k with amax = max|x|,
//     x_k = sx * (d0_k + d1_k/128 + d2_k/16384) + e_k,   |e_k| <= amax * 2^-22,
// three int8 digit planes that occupy three of the eight MMA columns (columns 4..6 hold a
// second activation row). Integer sums are exact; per group and row
//     y += scale * sx * (I0 + I1/128 + I2/16384) + bias * sum_k x_k
// is accumulated in f32.
//
// Mapping. A row block is 16*RT consecutive rows over the whole K. The K/64 groups are split
// over W consumer warps, J consecutive groups each, whose digit fragments stay in registers
// for the life of the CTA. A producer warp stages row blocks with 1-D bulk (TMA) copies, one
// per row so that rows can sit at a padded stride in shared memory (row stride = 8 words mod
// 32: the 8-byte fragment loads of a half-warp then hit 32 different banks), through a ring
// of stages handed over with full/empty mbarriers. Each warp leaves its partial sums for the
// block in a ring of buffers published through mbarriers; one warp (rotating) adds the W
// partials of every output in a fixed order, so results are deterministic.
#pragma once
#include "common.cuh"
#include "qmv.hpp"

#include <algorithm>
#include <map>
#include <mutex>
#include <tuple>

namespace lthn {

struct I8Args {
    const uint32_t* wq[2];
    const uint16_t* scales[2];
    const uint16_t* biases[2];
    const void* x;
    void* y;
    int64_t N, K;
    int x_dtype, y_dtype;
    int W;        // consumer warps; warp W is the producer
    int nblocks;  // row blocks
    int RS;       // shared-memory row stride in bytes
    int stg;      // ring stages (2..4)
    int bs_off, stage_off;  // byte offsets into dynamic shared memory
    int fuse_norm;          // 1: activations come from the fused residual RMSNorm prologue (nf)
    int ks, Gs;             // K slices (CTA c works on slice c % ks) and groups per slice
    int bits;               // 4 or 8 (8: plain matvec only, one byte per code, no unpack step)
    float* ypart;           // ks > 1: partial sums [ks][M][N] f32 instead of y
    NormFuse nf;
    float* const* push;     // npush > 0: f32 results go to these buffers (array in device memory) instead of y
    int npush;
    uint32_t* status;
};

__device__ __forceinline__ void mma_u8s8(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// first MMA of a group: accumulator input is constant zero (no register moves)
__device__ __forceinline__ void mma_u8s8_z(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                           uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
        : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0));
}

__device__ __forceinline__ float gelu_tanh_i8(float x) {
    const float k0 = 0.7978845608028654f, k1 = 0.044715f;
    return 0.5f * x * (1.0f + tanhf(k0 * (x + k1 * x * x * x)));
}

__device__ __forceinline__ float bf16f(uint16_t h) { return __uint_as_float((uint32_t)h << 16); }

// J groups per warp, RT 16-row tiles per row block, MT activation rows (1 or 2),
// FUSE != 0: two weight sets, output gelu_tanh(W1 x) * (W2 x). FUSE=1 stages 16 rows of each set
// per row block (short rows: fewer, fatter blocks); FUSE=2 stages 8 rows of each set as MMA rows
// 0-7 and 8-15, so a stage is as large as an unfused one (long rows: more blocks fit an SM).
// BITS = 8: a group of a row is 64 code bytes that go into the MMA as they are. The MMA's k
// index may be permuted freely as long as both operands agree, so thread t of a fragment takes the eight
// consecutive bytes 8t..8t+7 of a 32-code half group (one 8-byte load per row) and the activation digits sit in
// natural order.
template <int J, int RT, int MT, int FUSE, int BITS = 4>
__device__ __forceinline__ void qmv_i8_body(const I8Args& a) {
    static_assert(BITS == 4 || BITS == 8, "4-bit or 8-bit codes");
    constexpr int GB = BITS * 8;  // code bytes per group and row
    constexpr int SETS = FUSE == 1 ? 2 : 1;
    constexpr int OR = FUSE == 2 ? 8 : 16;  // output rows per row block
    constexpr int RB = 16 * RT;
    const int PR = 2 * a.stg;  // ring of partial-sum buffers, twice the stage count (see below)
    extern __shared__ __align__(128) unsigned char dsm[];
    pdl_trigger();
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int W = a.W;
    const int64_t K = a.K;
    // K may be cut into ks slices of Gs groups: CTA c streams slice c % ks of its row blocks and leaves
    // partial sums (small matrices then fill the GPU, long rows fit the shared-memory ring)
    const int G = (int)(K >> 6), Gs = a.Gs, ks = a.ks;
    const int slice = blockIdx.x % ks, cta = blockIdx.x / ks;
    const int rowbytes = Gs * GB, sbrow = Gs * 2, RS = a.RS;
    const int sb_bytes = (RB * sbrow + 15) & ~15;
    const int set_bytes = RB * RS + 2 * sb_bytes;
    const int stage_bytes = SETS * set_bytes;
    const int stg = a.stg;
    uint64_t* full = (uint64_t*)dsm;
    uint64_t* empty = full + 4;
    uint64_t* pfull = full + 8;                    // [PR], PR <= 8
    double* nsum = (double*)(dsm + 256);           // [2][16] cross-warp sums of the fused norm prologue
    float* part = (float*)(dsm + 512);             // [PR][W][SETS][RB*MT]
    unsigned char* Bs = dsm + a.bs_off;            // [W][MT][3][64] conversion scratch, digit bytes in fragment order
    unsigned char* stages = dsm + a.stage_off;
    const int stride = gridDim.x / ks;

    if (tid == 0) {
        for (int i = 0; i < 4; i++) { mbar_init(&full[i], ks > 1 ? 2 : 1); mbar_init(&empty[i], W); }
        for (int i = 0; i < PR; i++) mbar_init(&pfull[i], W);
        mbar_fence_init();
    }
    __syncthreads();

    if (warp >= W) {
        // ---- producer: weights do not depend on the previous kernel, start at once ------------
        if (warp > W) return;
        int it = 0;
        for (int b = cta; b < a.nblocks; b += stride, it++) {
            const int st = it % stg;
            if (!mbar_wait(&empty[st], ((it / stg) & 1) ^ 1)) { if (lane == 0) atomicOr(a.status, 32u); break; }
            unsigned char* sbase = stages + (size_t)st * stage_bytes;
            const int64_t row0 = (int64_t)b * OR;
            const int rows = FUSE == 2 ? 16 : (int)min((int64_t)RB, a.N - row0);  // a multiple of 16
            if (lane == 0) mbar_expect_tx(&full[st], (uint32_t)(SETS * rows * (rowbytes + (ks > 1 ? 0 : 2 * sbrow))));
            __syncwarp();
            if (FUSE == 2) {
                unsigned char* d = sbase;
                if (lane < 16) {
                    const int set = lane >> 3, r = lane & 7;
                    bulk_g2s(d + (size_t)lane * RS, (const unsigned char*)a.wq[set] + (row0 + r) * (K * BITS / 8), (uint32_t)rowbytes, &full[st]);
                } else if (lane < 20) {
                    const int set = lane & 1, which = (lane >> 1) & 1;  // which: 0 scales, 1 biases
                    const uint16_t* src = which ? a.biases[set] : a.scales[set];
                    bulk_g2s(d + (size_t)RB * RS + (which ? sb_bytes : 0) + (size_t)set * 8 * sbrow,
                             (const unsigned char*)src + row0 * sbrow, (uint32_t)(8 * sbrow), &full[st]);
                }
            }
#pragma unroll
            for (int s = 0; s < (FUSE == 2 ? 0 : SETS); s++) {
                unsigned char* d = sbase + (size_t)s * set_bytes;
                const unsigned char* wsrc = (const unsigned char*)a.wq[s] + (size_t)slice * rowbytes;
                for (int r = lane; r < rows; r += 32)
                    bulk_g2s(d + (size_t)r * RS, wsrc + (row0 + r) * (K * BITS / 8), (uint32_t)rowbytes, &full[st]);
                if (ks == 1) {
                    if (lane == 0)
                        bulk_g2s(d + (size_t)RB * RS, (const unsigned char*)a.scales[s] + row0 * sbrow, (uint32_t)(rows * sbrow), &full[st]);
                    if (lane == 1)
                        bulk_g2s(d + (size_t)RB * RS + sb_bytes, (const unsigned char*)a.biases[s] + row0 * sbrow, (uint32_t)(rows * sbrow), &full[st]);
                }
            }
            if (ks > 1) {
                // a slice of a scale row is too short and too oddly placed for a bulk copy: plain loads
                // (4 bytes each; G and Gs are even), published with a second arrival on the barrier
                const int wpr = Gs >> 1;  // words per row
#pragma unroll
                for (int s = 0; s < SETS; s++) {
                    unsigned char* d = sbase + (size_t)s * set_bytes;
                    uint32_t* ds = (uint32_t*)(d + (size_t)RB * RS);
                    uint32_t* db = (uint32_t*)(d + (size_t)RB * RS + sb_bytes);
                    for (int i = lane; i < rows * wpr; i += 32) {
                        const int r = i / wpr, w = i - r * wpr;
                        const int64_t e = (row0 + r) * G + (int64_t)slice * Gs;
                        ds[i] = __ldg((const uint32_t*)(a.scales[s] + e) + w);
                        db[i] = __ldg((const uint32_t*)(a.biases[s] + e) + w);
                    }
                }
                __syncwarp();
                if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(&full[st])) : "memory");
            }
        }
        return;
    }

    // ---- consumers: activations -> digit fragments (each warp converts the groups it owns) ----
    pdl_wait();
    const int gq = lane >> 2, t = lane & 3;
    // activations of the owned groups: lane holds elements 2*lane, 2*lane+1 of each group
    float xr[J][MT][2];
    if (!a.fuse_norm) {
#pragma unroll
        for (int j = 0; j < J; j++)
#pragma unroll
            for (int m = 0; m < MT; m++) {
                const int g = slice * Gs + warp * J + j;
                if (a.x_dtype == LTHN_DTYPE_BF16) {
                    const uint32_t v = __ldg((const uint32_t*)((const uint16_t*)a.x + (int64_t)m * K + (int64_t)g * 64) + lane);
                    xr[j][m][0] = __uint_as_float(v << 16);
                    xr[j][m][1] = __uint_as_float(v & 0xffff0000u);
                } else {
                    const float2 v = __ldg((const float2*)((const float*)a.x + (int64_t)m * K + (int64_t)g * 64) + lane);
                    xr[j][m][0] = v.x; xr[j][m][1] = v.y;
                }
            }
    } else {
        // fused residual RMSNorm pair (see NormFuse). The W consumer warps cover the whole vector
        // between them; sums of squares are f64, reduced over the warps through shared memory
        // with a named barrier that the producer warp does not join.
        const NormFuse& nf = a.nf;
        const int nthr = W * 32;
        if (nf.wait) {
            // tensor parallel: signal this exchange to the peers, wait for theirs (bounded)
            const PeerWait& pw = *nf.wait;  // in device memory
            uint32_t* seq_s = (uint32_t*)(dsm + 192);  // spare word of the barrier header
            if (tid == 0) *seq_s = *(volatile uint32_t*)&pw.ctr[0] + 1u;
            asm volatile("bar.sync 1, %0;" ::"r"(nthr) : "memory");
            const uint32_t seq = *seq_s;
            if (warp == 0 && lane < pw.t) {
                if (blockIdx.x == 0) {
                    __threadfence_system();
                    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(pw.flag_out[lane] + pw.rank), "r"(seq) : "memory");
                }
                bool ok = false;
                for (uint32_t it = 0; it < (1u << 21); ++it) {
                    uint32_t f;
                    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(f) : "l"(pw.flag_in + lane) : "memory");
                    if ((int32_t)(f - seq) >= 0) { ok = true; break; }
                    __nanosleep(it < 64 ? 20 : 500);
                }
                if (!ok) atomicOr(a.status, 256u);
            }
            asm volatile("bar.sync 1, %0;" ::"r"(nthr) : "memory");
            // the last CTA past this point advances the sequence number (every CTA read it above)
            if (tid == 0) {
                if (atomicAdd(&pw.ctr[1], 1u) == gridDim.x - 1) {
                    pw.ctr[1] = 0u;
                    __threadfence();
                    *(volatile uint32_t*)&pw.ctr[0] = seq;
                }
            }
        }
        float2 wn[J];
        float hv[J][MT][2];
#pragma unroll
        for (int j = 0; j < J; j++) {
            const int64_t e0 = (int64_t)(warp * J + j) * 64 + 2 * lane;
            wn[j] = __ldg((const float2*)(nf.w_next + e0));
#pragma unroll
            for (int m = 0; m < MT; m++) {
                const float2 v = *(const float2*)(nf.h_in + (int64_t)m * K + e0);
                hv[j][m][0] = v.x; hv[j][m][1] = v.y;
            }
        }
        double ss[MT];
        if (nf.a) {
            float2 wp[J];
#pragma unroll
            for (int m = 0; m < MT; m++) ss[m] = 0.0;
            if (nf.na == 1) {
#pragma unroll
                for (int j = 0; j < J; j++) {
                    const int64_t e0 = (int64_t)(warp * J + j) * 64 + 2 * lane;
                    wp[j] = __ldg((const float2*)(nf.w_post + e0));
#pragma unroll
                    for (int m = 0; m < MT; m++) {
                        const float2 v = *(const float2*)(nf.a + (int64_t)m * K + e0);
                        xr[j][m][0] = v.x; xr[j][m][1] = v.y;
                        ss[m] += (double)__fmul_rn(v.x, v.x);
                        ss[m] += (double)__fmul_rn(v.y, v.y);
                    }
                }
            } else {
                // tensor parallel: one partial vector per rank, added in rank order, one rank (one
                // batch of independent loads) at a time
#pragma unroll
                for (int j = 0; j < J; j++) {
                    const int64_t e0 = (int64_t)(warp * J + j) * 64 + 2 * lane;
                    wp[j] = __ldg((const float2*)(nf.w_post + e0));
#pragma unroll
                    for (int m = 0; m < MT; m++) {
                        const float2 v = *(const float2*)(nf.a + (int64_t)m * K + e0);
                        xr[j][m][0] = v.x; xr[j][m][1] = v.y;
                    }
                }
                for (int r = 1; r < nf.na; r++) {
                    const float* ar = nf.a + (int64_t)r * nf.a_stride;
#pragma unroll
                    for (int j = 0; j < J; j++) {
                        const int64_t e0 = (int64_t)(warp * J + j) * 64 + 2 * lane;
#pragma unroll
                        for (int m = 0; m < MT; m++) {
                            const float2 u = *(const float2*)(ar + (int64_t)m * K + e0);
                            xr[j][m][0] = __fadd_rn(xr[j][m][0], u.x);
                            xr[j][m][1] = __fadd_rn(xr[j][m][1], u.y);
                        }
                    }
                }
#pragma unroll
                for (int j = 0; j < J; j++)
#pragma unroll
                    for (int m = 0; m < MT; m++) {
                        ss[m] += (double)__fmul_rn(xr[j][m][0], xr[j][m][0]);
                        ss[m] += (double)__fmul_rn(xr[j][m][1], xr[j][m][1]);
                    }
            }
#pragma unroll
            for (int m = 0; m < MT; m++) {
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) ss[m] += __shfl_xor_sync(0xffffffffu, ss[m], o);
                if (lane == 0) nsum[m * 16 + warp] = ss[m];
            }
            asm volatile("bar.sync 1, %0;" ::"r"(nthr) : "memory");
            float rms[MT];
#pragma unroll
            for (int m = 0; m < MT; m++) {
                double tsum = 0.0;
                for (int w = 0; w < W; w++) tsum += nsum[m * 16 + w];
                rms[m] = fast_rms(tsum, nf.inv_width, nf.eps);
            }
            asm volatile("bar.sync 1, %0;" ::"r"(nthr) : "memory");
            FastDiv kd[MT];
#pragma unroll
            for (int m = 0; m < MT; m++) kd[m] = fast_div_by(rms[m]);
#pragma unroll
            for (int j = 0; j < J; j++) {
                const int64_t e0 = (int64_t)(warp * J + j) * 64 + 2 * lane;
#pragma unroll
                for (int m = 0; m < MT; m++) {
                    hv[j][m][0] = __fadd_rn(hv[j][m][0], __fmul_rn(fast_div(xr[j][m][0], kd[m]), wp[j].x));
                    hv[j][m][1] = __fadd_rn(hv[j][m][1], __fmul_rn(fast_div(xr[j][m][1], kd[m]), wp[j].y));
                    if (blockIdx.x == 0) *(float2*)(nf.h_out + (int64_t)m * K + e0) = make_float2(hv[j][m][0], hv[j][m][1]);
                }
            }
        }
#pragma unroll
        for (int m = 0; m < MT; m++) ss[m] = 0.0;
#pragma unroll
        for (int j = 0; j < J; j++)
#pragma unroll
            for (int m = 0; m < MT; m++) {
                ss[m] += (double)__fmul_rn(hv[j][m][0], hv[j][m][0]);
                ss[m] += (double)__fmul_rn(hv[j][m][1], hv[j][m][1]);
            }
#pragma unroll
        for (int m = 0; m < MT; m++) {
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) ss[m] += __shfl_xor_sync(0xffffffffu, ss[m], o);
            if (lane == 0) nsum[m * 16 + warp] = ss[m];
        }
        asm volatile("bar.sync 1, %0;" ::"r"(nthr) : "memory");
#pragma unroll
        for (int m = 0; m < MT; m++) {
            double tsum = 0.0;
            for (int w = 0; w < W; w++) tsum += nsum[m * 16 + w];
            const FastDiv k2 = fast_div_by(fast_rms(tsum, nf.inv_width, nf.eps));
#pragma unroll
            for (int j = 0; j < J; j++) {
                xr[j][m][0] = __fmul_rn(fast_div(hv[j][m][0], k2), wn[j].x);
                xr[j][m][1] = __fmul_rn(fast_div(hv[j][m][1], k2), wn[j].y);
            }
        }
    }
    // B fragments: column n = lane>>2 carries digit plane n&3 of activation row n>>2;
    // accumulator columns (2t, 2t+1) are planes (0,1) of row t>>1 for even t and (2, none) for odd t.
    uint32_t bfrag[J][2][2];
    float cg[J], xsb[J];
    {
        const int bm = gq >> 2, bp = gq & 3, dm = t >> 1;
        unsigned char* Bw = Bs + (size_t)warp * (MT * 192 + J * 32);  // this warp's scratch: [MT][3][64] digit bytes, then [J][4] constants
#pragma unroll
        for (int j = 0; j < J; j++) {
            float sx_d = 0.f, xs_d = 0.f;
#pragma unroll
            for (int m = 0; m < MT; m++) {
                const float xv[2] = {xr[j][m][0], xr[j][m][1]};
                // non-negative floats order like their bit patterns: one redux instead of five shuffles
                const float amax = __uint_as_float(__reduce_max_sync(0xffffffffu, __float_as_uint(fmaxf(fabsf(xv[0]), fabsf(xv[1])))));
                const float sx = amax * (1.0f / 127.0f);
                const float inv = amax > 0.f ? __fdividef(127.0f, amax) : 0.f;
                const float sx1 = sx * (1.0f / 128.0f);
                int isum = 0;
#pragma unroll
                for (int q = 0; q < 2; q++) {
                    const float x0 = xv[q];
                    const float d0 = rintf(x0 * inv);
                    const float r1 = fmaf(-d0, sx, x0);
                    const float d1 = rintf(r1 * inv * 128.0f);
                    const float r2 = fmaf(-d1, sx1, r1);
                    const float d2 = rintf(r2 * inv * 16384.0f);
                    const int i0 = (int)d0, i1 = (int)d1, i2 = (int)d2;
                    isum += i0 * 16384 + i1 * 128 + i2;
                    // element e of the group: word e>>3 of the row piece, nibble e&7. Thread t of a
                    // fragment owns words 2t (first MMA) and 2t+1 (second); even nibbles feed the
                    // low k half, odd nibbles the high k half.
                    const int e = 2 * lane + q;
                    const int off = BITS == 8 ? e : ((((e >> 3) & 1) * 4 + (e >> 4)) * 2 + (e & 1)) * 4 + ((e & 7) >> 1);
                    Bw[m * 192 + off] = (unsigned char)(i0 & 0xff);
                    Bw[m * 192 + 64 + off] = (unsigned char)(i1 & 0xff);
                    Bw[m * 192 + 128 + off] = (unsigned char)(i2 & 0xff);
                }
                isum = __reduce_add_sync(0xffffffffu, isum);
                if (m == dm) { sx_d = sx; xs_d = (float)isum * (sx * (1.0f / 16384.0f)); }
            }
            __syncwarp();
#pragma unroll
            for (int h = 0; h < 2; h++) {
                uint2 v = make_uint2(0u, 0u);
                if (bp < 3 && bm < MT) v = *(const uint2*)(Bw + bm * 192 + bp * 64 + (h * 4 + t) * 8);
                bfrag[j][h][0] = v.x;
                bfrag[j][h][1] = v.y;
            }
            __syncwarp();
            cg[j] = sx_d * ((t & 1) ? (1.0f / 2097152.0f) : (1.0f / 128.0f));
            xsb[j] = xs_d;
        }
    }

    // With many groups per warp the per-group constants (plane weight, activation sum) go to shared
    // memory, one pair per (group, t): measured on the lm_head shape, the loop with fewer live
    // registers runs 13 % faster (54.4 us against 63.0 us on the same GPU).
    constexpr bool GC_SMEM = J >= 6;
    const float2* gconst = (const float2*)(Bs + (size_t)warp * (MT * 192 + J * 32) + MT * 192) + t;
    if (GC_SMEM && gq == 0) {
#pragma unroll
        for (int j = 0; j < J; j++) ((float2*)(Bs + (size_t)warp * (MT * 192 + J * 32) + MT * 192))[j * 4 + t] = make_float2(cg[j], xsb[j]);
    }
    __syncwarp();

    constexpr uint32_t NIB = 0x0F0F0F0Fu;
    int it = 0;
    for (int b = cta; b < a.nblocks; b += stride, it++) {
        const int st = it % stg;
        if (!mbar_wait(&full[st], (it / stg) & 1)) { if (lane == 0) atomicOr(a.status, 64u); break; }
        const unsigned char* sbase = stages + (size_t)st * stage_bytes;
        float acc[SETS][RT][2], accb[SETS][RT];
#pragma unroll
        for (int s = 0; s < SETS; s++)
#pragma unroll
            for (int rt = 0; rt < RT; rt++) {
                acc[s][rt][0] = 0.f; acc[s][rt][1] = 0.f; accb[s][rt] = 0.f;
                const unsigned char* setp = sbase + (size_t)s * set_bytes;
                const unsigned char* rowp = setp + (size_t)(rt * 16 + gq) * RS + t * 8 + warp * J * GB;
                const uint16_t* sp = (const uint16_t*)(setp + (size_t)RB * RS) + (rt * 16 + gq) * Gs + warp * J;
                const uint16_t* bp = (const uint16_t*)(setp + (size_t)RB * RS + sb_bytes) + (rt * 16 + gq + 8 * (t & 1)) * Gs + warp * J;
#pragma unroll
                for (int j = 0; j < J; j++) {
                    int c[4];
                    if constexpr (BITS == 8) {
                        const uint2 wa0 = *(const uint2*)(rowp + j * 64), wb0 = *(const uint2*)(rowp + (size_t)8 * RS + j * 64);
                        const uint2 wa1 = *(const uint2*)(rowp + j * 64 + 32), wb1 = *(const uint2*)(rowp + (size_t)8 * RS + j * 64 + 32);
                        mma_u8s8_z(c, wa0.x, wb0.x, wa0.y, wb0.y, bfrag[j][0][0], bfrag[j][0][1]);
                        mma_u8s8(c, wa1.x, wb1.x, wa1.y, wb1.y, bfrag[j][1][0], bfrag[j][1][1]);
                    } else {
                        const uint2 wa = *(const uint2*)(rowp + j * 32);
                        const uint2 wb = *(const uint2*)(rowp + (size_t)8 * RS + j * 32);
                        mma_u8s8_z(c, wa.x & NIB, wb.x & NIB, (wa.x >> 4) & NIB, (wb.x >> 4) & NIB, bfrag[j][0][0], bfrag[j][0][1]);
                        mma_u8s8(c, wa.y & NIB, wb.y & NIB, (wa.y >> 4) & NIB, (wb.y >> 4) & NIB, bfrag[j][1][0], bfrag[j][1][1]);
                    }
                    const float s0 = bf16f(sp[j]), s1 = bf16f(sp[8 * Gs + j]);
                    const float2 gc = GC_SMEM ? gconst[j * 4] : make_float2(cg[j], xsb[j]);
                    const float f0 = (float)(c[0] * 128 + c[1]) * gc.x;
                    const float f1 = (float)(c[2] * 128 + c[3]) * gc.x;
                    acc[s][rt][0] = fmaf(s0, f0, acc[s][rt][0]);
                    acc[s][rt][1] = fmaf(s1, f1, acc[s][rt][1]);
                    accb[s][rt] = fmaf(bf16f(bp[j]), gc.y, accb[s][rt]);
                }
            }
        // this warp is done reading the stage: hand it back to the producer
        __syncwarp();
        if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(&empty[st])) : "memory");
        // Lanes t and t^1 hold the two plane halves of the same outputs; even t finishes row gq,
        // odd t row gq+8 (each also carries that row's bias term).
        const int pb = it % PR;
        float* pw = part + ((size_t)(pb * W + warp) * SETS) * (RB * MT);
#pragma unroll
        for (int s = 0; s < SETS; s++)
#pragma unroll
            for (int rt = 0; rt < RT; rt++) {
                const bool odd = t & 1;
                const float send = odd ? acc[s][rt][0] : acc[s][rt][1];
                const float recv = __shfl_xor_sync(0xffffffffu, send, 1);
                const float res = (odd ? acc[s][rt][1] : acc[s][rt][0]) + recv + accb[s][rt];
                const int m = t >> 1;
                if (m < MT) pw[(size_t)s * (RB * MT) + (rt * 16 + gq + 8 * (t & 1)) * MT + m] = res;
            }
        // No block-wide barrier: each warp publishes its partials on the buffer's mbarrier and moves
        // on; one warp (rotating with the block number) waits for all of them and adds the W
        // partials of every output in a fixed order. A warp can run at most stg blocks ahead of the
        // slowest one (the weight ring throttles it), so PR >= 2*stg buffers are never overwritten
        // while they are being summed.
        __syncwarp();
        if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(&pfull[pb])) : "memory");
        if (warp == it % W) {
            if (!mbar_wait(&pfull[pb], (it / PR) & 1)) { if (lane == 0) atomicOr(a.status, 128u); break; }
            for (int o = lane; o < OR * MT; o += 32) {
                const float* p0 = part + ((size_t)pb * W * SETS) * (RB * MT) + o;
                float v0 = 0.f, v1 = 0.f;
                for (int w = 0; w < W; w++) v0 += p0[(size_t)w * SETS * (RB * MT)];
                if (FUSE == 1) {
                    for (int w = 0; w < W; w++) v1 += p0[((size_t)w * SETS + 1) * (RB * MT)];
                    v0 = gelu_tanh_i8(v0) * v1;
                } else if (FUSE == 2) {
                    for (int w = 0; w < W; w++) v1 += p0[(size_t)w * SETS * (RB * MT) + 8 * MT];  // the up row of this gate row
                    v0 = gelu_tanh_i8(v0) * v1;
                }
                const int r = o / MT, m = o - r * MT;
                const int64_t row = (int64_t)b * OR + r;
                if (row < a.N) {
                    if (ks > 1) a.ypart[((int64_t)slice * MT + m) * a.N + row] = v0;
                    else if (a.npush) {
                        for (int p = 0; p < a.npush; p++) a.push[p][(int64_t)m * a.N + row] = v0;
                    } else if (a.y_dtype == LTHN_DTYPE_BF16) ((uint16_t*)a.y)[(int64_t)m * a.N + row] = f32_to_bf16_bits(v0);
                    else ((float*)a.y)[(int64_t)m * a.N + row] = v0;
                }
            }
        }
    }
}

// LB bounds the block size ((W+1)*32 threads). The small-block variant (up to 4 consumer warps,
// the long-stream configuration) asks for five blocks per SM, which holds it to 72 registers.
template <int J, int RT, int MT, int FUSE, int LB>
__global__ void __launch_bounds__(LB) qmv_i8_kernel(const I8Args a) { qmv_i8_body<J, RT, MT, FUSE>(a); }
template <int J, int RT, int MT, int FUSE>
__global__ void __launch_bounds__(160, 5) qmv_i8_kernel_small(const I8Args a) { qmv_i8_body<J, RT, MT, FUSE>(a); }

// 8-bit codes: one block per SM class only (the stages are twice as large, so two to four blocks fit an SM anyway)
template <int J, int MT, int FUSE, int LB>
__global__ void __launch_bounds__(LB) qmv_i8_b8_kernel(const I8Args a) { qmv_i8_body<J, 1, MT, FUSE, 8>(a); }

template <int J, int RT, int MT, int FUSE, int LB, int BITS = 4>
inline int32_t launch_i8_t(cudaStream_t st, const I8Args& a, const I8Plan& p) {
    static int attr_dev = -1;
    static std::mutex mu;  // guards attr_dev and occ_cache: entry points may be called from several host threads
    int dev = 0;
    LTHN_CUDA_TRY(cudaGetDevice(&dev));
    void (*kern)(const I8Args);
    if constexpr (BITS == 8) kern = qmv_i8_b8_kernel<J, MT, FUSE, LB>;
    else kern = LB == 160 ? qmv_i8_kernel_small<J, RT, MT, FUSE> : qmv_i8_kernel<J, RT, MT, FUSE, LB>;
    std::unique_lock<std::mutex> lk(mu);
    if (attr_dev != dev) {
        LTHN_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 224 * 1024));
        LTHN_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared));
        attr_dev = dev;
    }
    static std::map<std::tuple<int, int, size_t>, int> occ_cache;
    const auto key = std::make_tuple(dev, p.threads, p.smem);
    auto it = occ_cache.find(key);
    int occ;
    if (it == occ_cache.end()) {
        LTHN_CUDA_TRY(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, kern, p.threads, p.smem));
        if (occ < 1) return fail(LTHN_ERR_CUDA, "affine_qmv: integer tensor-core kernel does not fit on an SM");
        occ_cache[key] = occ;
    } else {
        occ = it->second;
    }
    lk.unlock();
    int sms = 148;
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const int grid = std::max(1, std::min(p.nblocks, sms * occ / p.ks)) * p.ks;
    LTHN_CUDA_TRY(launch_k(kern, dim3(grid), dim3(p.threads), p.smem, st, a));
    return LTHN_OK;
}

template <int J, int LB>
inline int32_t launch_i8_j(cudaStream_t st, const I8Args& a, const I8Plan& p, int M, int fuse) {
    // one 16-row tile per row block: taller blocks measured slower (fewer blocks per SM)
    if (fuse == 1) return M == 1 ? launch_i8_t<J, 1, 1, 1, LB>(st, a, p) : launch_i8_t<J, 1, 2, 1, LB>(st, a, p);
    if (fuse == 2) return M == 1 ? launch_i8_t<J, 1, 1, 2, LB>(st, a, p) : launch_i8_t<J, 1, 2, 2, LB>(st, a, p);
    if (M == 1) return launch_i8_t<J, 1, 1, 0, LB>(st, a, p);
    return launch_i8_t<J, 1, 2, 0, LB>(st, a, p);
}

// 8-bit codes: J in {2, 3, 4, 6, 9, 12}, block classes of up to 8 and up to 16 consumer warps
template <int J, int LB>
inline int32_t launch_i8_b8_j(cudaStream_t st, const I8Args& a, const I8Plan& p, int M, int fuse) {
    if (fuse == 1) return M == 1 ? launch_i8_t<J, 1, 1, 1, LB, 8>(st, a, p) : launch_i8_t<J, 1, 2, 1, LB, 8>(st, a, p);
    if (fuse == 2) return M == 1 ? launch_i8_t<J, 1, 1, 2, LB, 8>(st, a, p) : launch_i8_t<J, 1, 2, 2, LB, 8>(st, a, p);
    return M == 1 ? launch_i8_t<J, 1, 1, 0, LB, 8>(st, a, p) : launch_i8_t<J, 1, 2, 0, LB, 8>(st, a, p);
}
template <int J>
int32_t launch_i8_b8(cudaStream_t st, const I8Args& a, const I8Plan& p, int M, int fuse) {
    if (p.W <= 8) return launch_i8_b8_j<J, 288>(st, a, p, M, fuse);
    if constexpr (J <= 9) return launch_i8_b8_j<J, 544>(st, a, p, M, fuse);
    return fail(LTHN_ERR_INVALID, "affine_qmv: no 8-bit integer tensor-core instantiation for this plan");
}

// block-size classes: up to 4, 8 and 16 consumer warps (plus the producer warp)
template <int J>
int32_t launch_i8_w(cudaStream_t st, const I8Args& a, const I8Plan& p, int M, int fuse) {
    if (p.W <= 4) return launch_i8_j<J, 160>(st, a, p, M, fuse);
    if (p.W <= 8) return launch_i8_j<J, 288>(st, a, p, M, fuse);
    if constexpr (J <= 9) return launch_i8_j<J, 544>(st, a, p, M, fuse);
    return fail(LTHN_ERR_INVALID, "affine_qmv: no integer tensor-core instantiation for this plan");
}


}  // namespace lthn
