// qmv_dp4a.cu — affine_qmv for one or two activation rows (the batch-1 decode
// matvec), written for B200 (sm_100a). Integer dot products, no tensor cores.
//
// Why not the tensor cores here: at batch 1 an MMA wastes 7/8 of its columns, and
// on B200 the mma.sync path retires roughly one m16n8k16 per 8 SM cycles, which
// caps a tensor-core GEMV near half of HBM bandwidth (measured). dp4a does four
// 8-bit multiply-adds per lane per instruction and unpacking eight 4-bit codes
// to bytes costs three logic ops, so the whole dequant-dot needs about 45 issue
// slots per 16 weight bytes per lane - under half the SM's issue rate at full
// HBM speed.
//
// Arithmetic. Activations are converted once per CTA to block fixed point: for
// each quantisation group g (64 consecutive k) with amax = max|x|,
//     x_k = sx * (d0_k + d1_k/128 + d2_k/16384) + e_k,  |e_k| <= amax * 2^-22,
// with three int8 digit planes d0,d1,d2 (|d0|<=127, |d1|,|d2|<=65). Then
//     sum_k code_k * x_k = (sx/16384) * (16384*I0 + 128*I1 + I2),  I_p = sum code*d_p
// is exact integer arithmetic (dp4a accumulates in s32), and per group
//     y += scale * (sx' * I) + bias * (sx' * sum_k D_k)
// in f32. The activation error bound (2^-22 of the group maximum) is below the
// f32 rounding of the group maximum itself; all accumulation across groups is f32.
//
// Mapping. A row of K codes is K/32 "half groups" of 16 bytes. T_row = K/(32*J)
// threads cooperate on a row, thread u owning half groups u, u+T_row, ... (J of
// them), so a row is read as consecutive 16-byte loads. A CTA has S row slots
// (S*T_row threads) and is persistent: it converts its activations once into
// registers (24 registers per half group) and then streams row blocks of S*R
// rows, R rows per thread in flight plus the next block prefetched. Partial sums
// of the T_row threads of a row meet in shared memory (double buffered, one
// __syncthreads per row block) and are reduced in a fixed order by one warp per
// output, so results are deterministic.
#include "common.cuh"
#include "qmv.hpp"

#include <algorithm>
#include <map>
#include <tuple>

namespace lthn {

struct Dp4aArgs {
    const uint32_t* wq[2];
    const uint16_t* scales[2];
    const uint16_t* biases[2];
    const void* x;
    void* y;
    int64_t N, K;
    int x_dtype, y_dtype;
    int T_row, S, nblocks;
};

__device__ __forceinline__ int dp4a_ss(int a, int b, int c) { return __dp4a(a, b, c); }

__device__ __forceinline__ float gelu_tanh_dev(float x) {
    const float k0 = 0.7978845608028654f, k1 = 0.044715f;
    return 0.5f * x * (1.0f + tanhf(k0 * (x + k1 * x * x * x)));
}

// J half groups per thread, R rows per thread per block, MT activation rows,
// FUSE=1: two weight sets, output gelu_tanh(W1 x) * (W2 x).
template <int J, int R, int MT, int FUSE>
__global__ void __launch_bounds__(384) qmv_dp4a_kernel(const Dp4aArgs a) {
    constexpr int SETS = FUSE ? 2 : 1;
    extern __shared__ float part[];  // [2][SETS*S*R*MT][T_row]
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nwarps = blockDim.x >> 5;
    const int T_row = a.T_row;
    const int slot = tid / T_row, u = tid - slot * T_row;
    const bool active = slot < a.S;
    const int64_t K = a.K;

    // ---- activations -> three int8 digit planes per owned half group ---------------
    int X[MT][J][3][8];
    float sxp[MT][J], xq[MT][J];
#pragma unroll
    for (int m = 0; m < MT; m++)
#pragma unroll
        for (int j = 0; j < J; j++) {
            const int hg = (active ? u : 0) + j * T_row;
            float xv[32];
            if (a.x_dtype == LTHN_DTYPE_BF16) {
                const uint4* p = (const uint4*)((const uint16_t*)a.x + (int64_t)m * K + (int64_t)hg * 32);
#pragma unroll
                for (int q = 0; q < 4; q++) {
                    const uint4 v = __ldg(p + q);
                    const uint32_t ww[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
                    for (int e = 0; e < 4; e++) {
                        xv[q * 8 + e * 2] = __uint_as_float(ww[e] << 16);
                        xv[q * 8 + e * 2 + 1] = __uint_as_float(ww[e] & 0xffff0000u);
                    }
                }
            } else {
                const float4* p = (const float4*)((const float*)a.x + (int64_t)m * K + (int64_t)hg * 32);
#pragma unroll
                for (int q = 0; q < 8; q++) {
                    const float4 v = __ldg(p + q);
                    xv[q * 4] = v.x; xv[q * 4 + 1] = v.y; xv[q * 4 + 2] = v.z; xv[q * 4 + 3] = v.w;
                }
            }
            float amax = 0.f;
#pragma unroll
            for (int e = 0; e < 32; e++) amax = fmaxf(amax, fabsf(xv[e]));
            // the other half of this quantisation group lives in the neighbouring thread
            amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
            const float sx = amax * (1.0f / 127.0f);
            const float inv = amax > 0.f ? 127.0f / amax : 0.f;
            const float sx1 = sx * (1.0f / 128.0f);
            int isum = 0;
#pragma unroll
            for (int p = 0; p < 3; p++)
#pragma unroll
                for (int w8 = 0; w8 < 8; w8++) X[m][j][p][w8] = 0;
#pragma unroll
            for (int e = 0; e < 32; e++) {
                const float x0 = xv[e];
                const float d0 = rintf(x0 * inv);
                const float r1 = fmaf(-d0, sx, x0);
                const float d1 = rintf(r1 * inv * 128.0f);
                const float r2 = fmaf(-d1, sx1, r1);
                const float d2 = rintf(r2 * inv * 16384.0f);
                const int i0 = (int)d0, i1 = (int)d1, i2 = (int)d2;
                isum += i0 * 16384 + i1 * 128 + i2;
                // byte position inside the word pair: even k -> bytes of "even" reg, odd k -> "odd" reg
                const int word = e >> 3, pos = e & 7;
                const int reg = word * 2 + (pos & 1), sh = (pos >> 1) * 8;
                X[m][j][0][reg] |= (i0 & 0xff) << sh;
                X[m][j][1][reg] |= (i1 & 0xff) << sh;
                X[m][j][2][reg] |= (i2 & 0xff) << sh;
            }
            sxp[m][j] = sx * (1.0f / 16384.0f);
            xq[m][j] = (float)isum * sxp[m][j];
        }

    // ---- persistent loop over row blocks ----------------------------------------
    const int RB = a.S * R;
    const int64_t wpr = K >> 3;
    const int gpr = (int)(K >> 6);
    uint4 wcur[SETS][R][J], wnxt[SETS][R][J];
    uint32_t sbcur[SETS][R][J], sbnxt[SETS][R][J];

    auto load_block = [&](int b, uint4 (&w)[SETS][R][J], uint32_t (&sb)[SETS][R][J]) {
#pragma unroll
        for (int s = 0; s < SETS; s++)
#pragma unroll
            for (int r = 0; r < R; r++) {
                int64_t row = (int64_t)b * RB + slot * R + r;
                if (row >= a.N) row = a.N - 1;
#pragma unroll
                for (int j = 0; j < J; j++) {
                    const int hg = u + j * T_row;
                    w[s][r][j] = __ldg((const uint4*)(a.wq[s] + row * wpr + (int64_t)hg * 4));
                    const int64_t gi = row * gpr + (hg >> 1);
                    sb[s][r][j] = (uint32_t)__ldg(a.scales[s] + gi) | ((uint32_t)__ldg(a.biases[s] + gi) << 16);
                }
            }
    };

    int b = blockIdx.x;
    if (active && b < a.nblocks) load_block(b, wcur, sbcur);
    const int nout = a.S * R * MT;  // outputs per block per set
    int buf = 0;
    for (; b < a.nblocks; b += gridDim.x) {
        const int bn = b + gridDim.x;
        if (active && bn < a.nblocks) load_block(bn, wnxt, sbnxt);
        if (active) {
#pragma unroll
            for (int s = 0; s < SETS; s++)
#pragma unroll
                for (int r = 0; r < R; r++) {
                    float acc[MT];
#pragma unroll
                    for (int m = 0; m < MT; m++) acc[m] = 0.f;
#pragma unroll
                    for (int j = 0; j < J; j++) {
                        const uint4 w = wcur[s][r][j];
                        const uint32_t ww[4] = {w.x, w.y, w.z, w.w};
                        int ev[4], od[4];
#pragma unroll
                        for (int i = 0; i < 4; i++) {
                            ev[i] = (int)(ww[i] & 0x0F0F0F0Fu);
                            od[i] = (int)((ww[i] >> 4) & 0x0F0F0F0Fu);
                        }
                        const float sc = __uint_as_float(sbcur[s][r][j] << 16);
                        const float bi = __uint_as_float(sbcur[s][r][j] & 0xffff0000u);
#pragma unroll
                        for (int m = 0; m < MT; m++) {
                            int i0 = 0, i1 = 0, i2 = 0;
#pragma unroll
                            for (int i = 0; i < 4; i++) {
                                i0 = dp4a_ss(ev[i], X[m][j][0][2 * i], i0);
                                i0 = dp4a_ss(od[i], X[m][j][0][2 * i + 1], i0);
                                i1 = dp4a_ss(ev[i], X[m][j][1][2 * i], i1);
                                i1 = dp4a_ss(od[i], X[m][j][1][2 * i + 1], i1);
                                i2 = dp4a_ss(ev[i], X[m][j][2][2 * i], i2);
                                i2 = dp4a_ss(od[i], X[m][j][2][2 * i + 1], i2);
                            }
                            const int itot = i0 * 16384 + i1 * 128 + i2;
                            const float f = (float)itot * sxp[m][j];
                            acc[m] = fmaf(sc, f, acc[m]);
                            acc[m] = fmaf(bi, xq[m][j], acc[m]);
                        }
                    }
#pragma unroll
                    for (int m = 0; m < MT; m++)
                        part[((size_t)buf * SETS * nout + (size_t)s * nout + (slot * R + r) * MT + m) * T_row + u] = acc[m];
                }
        }
        __syncthreads();
        // one warp per output: fixed-order sum over the T_row partials
        for (int o = warp; o < nout; o += nwarps) {
            float v[SETS];
#pragma unroll
            for (int s = 0; s < SETS; s++) {
                const float* src = part + ((size_t)buf * SETS * nout + (size_t)s * nout + o) * T_row;
                float t = 0.f;
                for (int uu = lane; uu < T_row; uu += 32) t += src[uu];
                v[s] = warp_sum(t);
            }
            if (lane == 0) {
                const int m = o % MT, sr = o / MT;  // sr = slot*R + r
                const int64_t row = (int64_t)b * RB + sr;
                if (row < a.N) {
                    float out = v[0];
                    if (FUSE) out = gelu_tanh_dev(v[0]) * v[SETS - 1];
                    if (a.y_dtype == LTHN_DTYPE_BF16) ((uint16_t*)a.y)[(int64_t)m * a.N + row] = f32_to_bf16_bits(out);
                    else ((float*)a.y)[(int64_t)m * a.N + row] = out;
                }
            }
        }
        buf ^= 1;
        if (bn < a.nblocks) {
#pragma unroll
            for (int s = 0; s < SETS; s++)
#pragma unroll
                for (int r = 0; r < R; r++)
#pragma unroll
                    for (int j = 0; j < J; j++) { wcur[s][r][j] = wnxt[s][r][j]; sbcur[s][r][j] = sbnxt[s][r][j]; }
        }
    }
}

// ---- host side --------------------------------------------------------------------

bool dp4a_plan(int64_t N, int64_t K, int M, int fuse, int force_r, Dp4aPlan* p) {
    if (M < 1 || M > 2 || K % 64 != 0 || N < 1) return false;
    const int hg = (int)(K / 32);
    int J = 0;
    for (int cand : {1, 2, 3, 4}) {
        if (hg % cand) continue;
        const int t = hg / cand;
        if (t % 2 == 0 && t <= 352) { J = cand; break; }
    }
    if (!J) return false;
    const int T_row = hg / J;
    int S = std::max(1, 288 / T_row);
    S = std::min(S, 64);
    // rows per thread: large matrices amortise the reduction, small ones want every SM busy
    int R = 4;
    if (M == 2 || fuse) R = 2;
    while (R > 1 && (N + (int64_t)S * R - 1) / ((int64_t)S * R) < 2 * 148) R >>= 1;
    if (force_r > 0) R = force_r;
    if ((M == 2 || fuse) && R > 2) R = 2;
    if (J >= 3 && R > 2) R = 2;
    if (J >= 3 && (M == 2 || fuse)) R = 1;
    p->J = J; p->R = R; p->T_row = T_row; p->S = S;
    p->threads = (S * T_row + 31) / 32 * 32;
    if (p->threads > 384) return false;
    p->nblocks = (int)((N + (int64_t)S * R - 1) / ((int64_t)S * R));
    p->smem = (size_t)2 * (fuse ? 2 : 1) * S * R * M * T_row * sizeof(float);
    return p->smem <= 160 * 1024;
}

template <int J, int R, int MT, int FUSE>
static int32_t launch_dp4a_t(cudaStream_t st, const Dp4aArgs& a, const Dp4aPlan& p) {
    static int cached_dev = -1, cached_occ = 0;
    static size_t cached_smem = 0;
    int dev = 0;
    LTHN_CUDA_TRY(cudaGetDevice(&dev));
    auto kern = qmv_dp4a_kernel<J, R, MT, FUSE>;
    if (cached_dev != dev || cached_smem < p.smem) {
        LTHN_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024));
        cached_dev = dev;
        cached_smem = 160 * 1024;
        cached_occ = 0;
    }
    // occupancy depends on the block size and shared memory of this launch
    static std::map<std::tuple<int, int, size_t>, int> occ_cache;
    const auto key = std::make_tuple(dev, p.threads, p.smem);
    auto it = occ_cache.find(key);
    int occ;
    if (it == occ_cache.end()) {
        LTHN_CUDA_TRY(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, kern, p.threads, p.smem));
        if (occ < 1) return fail(LTHN_ERR_CUDA, "affine_qmv: dp4a kernel does not fit on an SM");
        occ_cache[key] = occ;
    } else {
        occ = it->second;
    }
    (void)cached_occ;
    int sms = 148;
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const int grid = std::min(p.nblocks, sms * occ);
    kern<<<grid, p.threads, p.smem, st>>>(a);
    LTHN_CUDA_TRY(cudaGetLastError());
    return LTHN_OK;
}

int32_t dp4a_launch(cudaStream_t st, const QmvCall& c, const Dp4aPlan& p) {
    Dp4aArgs a{};
    a.wq[0] = c.wq; a.scales[0] = c.scales; a.biases[0] = c.biases;
    a.wq[1] = c.wq2; a.scales[1] = c.scales2; a.biases[1] = c.biases2;
    a.x = c.x; a.y = c.y; a.N = c.N; a.K = c.K; a.x_dtype = c.x_dtype; a.y_dtype = c.y_dtype;
    a.T_row = p.T_row; a.S = p.S; a.nblocks = p.nblocks;
    const int fuse = c.wq2 ? 1 : 0;
#define LTHN_DP4A(JJ, RR, MM, FF) \
    if (p.J == JJ && p.R == RR && c.M == MM && fuse == FF) return launch_dp4a_t<JJ, RR, MM, FF>(st, a, p);
    LTHN_DP4A(1, 4, 1, 0) LTHN_DP4A(1, 2, 1, 0) LTHN_DP4A(1, 1, 1, 0)
    LTHN_DP4A(2, 4, 1, 0) LTHN_DP4A(2, 2, 1, 0) LTHN_DP4A(2, 1, 1, 0)
    LTHN_DP4A(3, 2, 1, 0) LTHN_DP4A(3, 1, 1, 0) LTHN_DP4A(4, 2, 1, 0) LTHN_DP4A(4, 1, 1, 0)
    LTHN_DP4A(1, 2, 2, 0) LTHN_DP4A(1, 1, 2, 0) LTHN_DP4A(2, 2, 2, 0) LTHN_DP4A(2, 1, 2, 0)
    LTHN_DP4A(3, 1, 2, 0) LTHN_DP4A(4, 1, 2, 0)
    LTHN_DP4A(1, 2, 1, 1) LTHN_DP4A(1, 1, 1, 1) LTHN_DP4A(2, 2, 1, 1) LTHN_DP4A(2, 1, 1, 1)
    LTHN_DP4A(3, 1, 1, 1) LTHN_DP4A(4, 1, 1, 1)
#undef LTHN_DP4A
    return fail(LTHN_ERR_INVALID, "affine_qmv: no dp4a instantiation for this plan");
}

}  // namespace lthn
