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
// Mapping. A row of K codes is K/64 groups of 32 bytes. T_row = K/(64*J) threads
// cooperate on a row, thread u owning groups u, u+T_row, ... (J of them), so a row
// is read as consecutive 32-byte pieces. A CTA has S row slots (S*T_row threads) and
// is persistent: it converts its activations once into registers (48 registers per
// group) and then streams row blocks of S*R rows, R rows per thread in flight plus
// the next block prefetched into a second register set. The partial sums of a row's
// threads are folded inside each quad with shuffles, meet in shared memory (double
// in a ring published through mbarriers, no block-wide barrier) and are added in a fixed
// order by one thread per output, so results are deterministic.
#include "common.cuh"
#include "qmv.hpp"

#include <algorithm>
#include <map>
#include <mutex>
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
    int part_bytes;    // bytes of the reduction area at the start of dynamic shared memory (16-byte multiple)
    int cons_threads;  // consumer threads (multiple of 32); one more warp is the producer
    uint32_t* status;
};

__device__ __forceinline__ int dp4a_ss(int a, int b, int c) { return __dp4a(a, b, c); }

__device__ __forceinline__ float gelu_tanh_dev(float x) {
    const float k0 = 0.7978845608028654f, k1 = 0.044715f;
    return 0.5f * x * (1.0f + tanhf(k0 * (x + k1 * x * x * x)));
}

// J groups per thread, R rows per thread per block, MT activation rows,
// FUSE=1: two weight sets, output gelu_tanh(W1 x) * (W2 x).
// A thread owns whole quantisation groups (64 codes = two 16-byte loads), so scale, bias
// and the integer-to-float step are paid once per 32 weight bytes. T_row = K/(64*J) threads
// share a row; T_row is a multiple of 4 so the four lanes of a quad always belong to one row
// and V = SETS*R*MT partial sums per lane are folded with a V-value butterfly (2 shuffles per
// level) before one lane per quad stores to shared memory.
template <int V>
__device__ __forceinline__ float quad_fold(float (&v)[V], int lane) {
    if (V == 4) {
        const bool hi = lane & 2;
        const float sa = hi ? v[0] : v[2], sb = hi ? v[1] : v[3];
        float ka = hi ? v[2] : v[0], kb = hi ? v[3] : v[1];
        ka += __shfl_xor_sync(0xffffffffu, sa, 2);
        kb += __shfl_xor_sync(0xffffffffu, sb, 2);
        const bool odd = lane & 1;
        const float send = odd ? ka : kb;
        float keep = odd ? kb : ka;
        keep += __shfl_xor_sync(0xffffffffu, send, 1);
        return keep;  // lane (b1,b0) of the quad holds value index 2*b1+b0
    } else if (V == 2) {
        const bool odd = lane & 1;
        const float send = odd ? v[0] : v[1];
        float keep = odd ? v[1] : v[0];
        keep += __shfl_xor_sync(0xffffffffu, send, 1);
        keep += __shfl_xor_sync(0xffffffffu, keep, 2);
        return keep;  // lanes with b0 = i hold value index i
    } else {
        float keep = v[0];
        keep += __shfl_xor_sync(0xffffffffu, keep, 1);
        keep += __shfl_xor_sync(0xffffffffu, keep, 2);
        return keep;
    }
}

template <int J, int R, int MT, int FUSE>
__global__ void __launch_bounds__(384) qmv_dp4a_kernel(const Dp4aArgs a) {
    constexpr int SETS = FUSE ? 2 : 1;
    constexpr int V = SETS * R * MT;
    static_assert(V == 1 || V == 2 || V == 4, "1, 2 or 4 partial sums per lane");
    extern __shared__ __align__(16) unsigned char dsm[];
    pdl_trigger();
    const int tid = threadIdx.x, lane = tid & 31;
    const int T_row = a.T_row, T4 = T_row >> 2;
    const int slot = tid / T_row, u = tid - slot * T_row;
    const bool active = slot < a.S;
    const int64_t K = a.K;

    // ---- persistent loop over row blocks, tiles staged by bulk (TMA) copies ------------------
    // A row block (RB consecutive rows) is contiguous in each of the three tensors, so one
    // elected lane of a dedicated producer warp fetches it with three 1-D bulk copies per
    // weight set into a ring of STG shared-memory stages, STG-1 blocks ahead of the
    // consumers; full/empty mbarriers hand the stages over. Consumer threads then read their
    // own 32-byte pieces and bf16 scale/bias with plain shared loads: no per-thread global
    // addressing, no registers spent on prefetch.
    constexpr int STG = 4;
    const int RB = a.S * R;
    const int G = (int)(K >> 6);
    const int rowbytes = (int)(K >> 1), sbrow = G * 2;
    const int codes_bytes = RB * rowbytes;              // multiple of 16
    const int sb_bytes = (RB * sbrow + 15) & ~15;       // section size, 16-byte aligned
    const int set_bytes = codes_bytes + 2 * sb_bytes;
    const int stage_bytes = SETS * set_bytes;
    constexpr int PR = 8;  // ring of partial-sum buffers; must be at least 2*STG (see below)
    float* part = (float*)dsm;                                               // [PR][V*S][T4]
    uint64_t* full = (uint64_t*)(dsm + a.part_bytes);
    uint64_t* empty = full + STG;
    uint64_t* pfull = empty + STG;                                           // [PR]
    unsigned char* stages = dsm + a.part_bytes + 128;
    const int ncons = a.cons_threads;                    // consumer threads (multiple of 32)
    const bool producer_warp = tid >= ncons;
    const int stride = gridDim.x;

    if (tid == 0) {
        for (int i = 0; i < STG; i++) { mbar_init(&full[i], 1); mbar_init(&empty[i], ncons >> 5); }
        for (int i = 0; i < PR; i++) mbar_init(&pfull[i], ncons >> 5);
        mbar_fence_init();
    }
    __syncthreads();

    if (producer_warp) {
        int it = 0;
        for (int b = blockIdx.x; b < a.nblocks; b += stride, it++) {
            const int st = it % STG;
            if (!mbar_wait(&empty[st], ((it / STG) & 1) ^ 1)) { if (lane == 0) atomicOr(a.status, 32u); break; }
            unsigned char* sbase = stages + (size_t)st * stage_bytes;
            const int64_t row0 = (int64_t)b * RB;
            const int rows = (int)min((int64_t)RB, a.N - row0);
            const bool bulk_ok = rows == RB;
            if (bulk_ok) {
                if (lane == 0) {
                    mbar_expect_tx(&full[st], (uint32_t)(SETS * (codes_bytes + 2 * RB * sbrow)));
#pragma unroll
                    for (int s = 0; s < SETS; s++) {
                        unsigned char* d = sbase + (size_t)s * set_bytes;
                        bulk_g2s(d, (const unsigned char*)a.wq[s] + row0 * rowbytes, (uint32_t)codes_bytes, &full[st]);
                        bulk_g2s(d + codes_bytes, (const unsigned char*)a.scales[s] + row0 * sbrow, (uint32_t)(RB * sbrow), &full[st]);
                        bulk_g2s(d + codes_bytes + sb_bytes, (const unsigned char*)a.biases[s] + row0 * sbrow, (uint32_t)(RB * sbrow), &full[st]);
                    }
                }
            } else {
                // last, partial block: plain copies by the producer warp (sizes are multiples of 8 bytes)
#pragma unroll
                for (int s = 0; s < SETS; s++) {
                    unsigned char* d = sbase + (size_t)s * set_bytes;
                    const uint2* src = (const uint2*)((const unsigned char*)a.wq[s] + row0 * rowbytes);
                    for (int i = lane; i < rows * rowbytes / 8; i += 32) ((uint2*)d)[i] = __ldg(src + i);
                    const uint2* ss = (const uint2*)((const unsigned char*)a.scales[s] + row0 * sbrow);
                    const uint2* bs = (const uint2*)((const unsigned char*)a.biases[s] + row0 * sbrow);
                    for (int i = lane; i < rows * sbrow / 8; i += 32) {
                        ((uint2*)(d + codes_bytes))[i] = __ldg(ss + i);
                        ((uint2*)(d + codes_bytes + sb_bytes))[i] = __ldg(bs + i);
                    }
                }
                __syncwarp();
                if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(&full[st])) : "memory");
            }
        }
        return;
    }

    // ---- consumers ----------------------------------------------------------------------------
    // (the producer is already fetching the first row blocks - weights do not depend on the
    // previous kernel - while the consumers wait for it and convert the activations)
    pdl_wait();
    // ---- activations -> three int8 digit planes per owned group -------------------------
    int X[MT][J][3][16];
    float sxp[MT][J], xq[MT][J];
#pragma unroll
    for (int m = 0; m < MT; m++)
#pragma unroll
        for (int j = 0; j < J; j++) {
            const int g = (active ? u : 0) + j * T_row;
            float xv[64];
            if (a.x_dtype == LTHN_DTYPE_BF16) {
                const uint4* p = (const uint4*)((const uint16_t*)a.x + (int64_t)m * K + (int64_t)g * 64);
#pragma unroll
                for (int q = 0; q < 8; q++) {
                    const uint4 v = __ldg(p + q);
                    const uint32_t ww[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
                    for (int e = 0; e < 4; e++) {
                        xv[q * 8 + e * 2] = __uint_as_float(ww[e] << 16);
                        xv[q * 8 + e * 2 + 1] = __uint_as_float(ww[e] & 0xffff0000u);
                    }
                }
            } else {
                const float4* p = (const float4*)((const float*)a.x + (int64_t)m * K + (int64_t)g * 64);
#pragma unroll
                for (int q = 0; q < 16; q++) {
                    const float4 v = __ldg(p + q);
                    xv[q * 4] = v.x; xv[q * 4 + 1] = v.y; xv[q * 4 + 2] = v.z; xv[q * 4 + 3] = v.w;
                }
            }
            float amax = 0.f;
#pragma unroll
            for (int e = 0; e < 64; e++) amax = fmaxf(amax, fabsf(xv[e]));
            const float sx = amax * (1.0f / 127.0f);
            const float inv = amax > 0.f ? __fdividef(127.0f, amax) : 0.f;
            const float sx1 = sx * (1.0f / 128.0f);
            int isum = 0;
#pragma unroll
            for (int p = 0; p < 3; p++)
#pragma unroll
                for (int w8 = 0; w8 < 16; w8++) X[m][j][p][w8] = 0;
#pragma unroll
            for (int e = 0; e < 64; e++) {
                const float x0 = xv[e];
                const float d0 = rintf(x0 * inv);
                const float r1 = fmaf(-d0, sx, x0);
                const float d1 = rintf(r1 * inv * 128.0f);
                const float r2 = fmaf(-d1, sx1, r1);
                const float d2 = rintf(r2 * inv * 16384.0f);
                const int i0 = (int)d0, i1 = (int)d1, i2 = (int)d2;
                isum += i0 * 16384 + i1 * 128 + i2;
                // even k -> bytes of the word's "even" register, odd k -> its "odd" register
                const int word = e >> 3, pos = e & 7;
                const int reg = word * 2 + (pos & 1), sh = (pos >> 1) * 8;
                X[m][j][0][reg] |= (i0 & 0xff) << sh;
                X[m][j][1][reg] |= (i1 & 0xff) << sh;
                X[m][j][2][reg] |= (i2 & 0xff) << sh;
            }
            sxp[m][j] = sx * (1.0f / 16384.0f);
            xq[m][j] = (float)isum * sxp[m][j];
        }

    int it = 0;
    for (int b = blockIdx.x; b < a.nblocks; b += stride, it++) {
        const int st = it % STG;
        if (!mbar_wait(&full[st], (it / STG) & 1)) { if (lane == 0) atomicOr(a.status, 64u); break; }
        const unsigned char* sbase = stages + (size_t)st * stage_bytes;
        float acc[V];
#pragma unroll
        for (int i = 0; i < V; i++) acc[i] = 0.f;
        if (active) {
#pragma unroll
            for (int s = 0; s < SETS; s++)
#pragma unroll
                for (int r = 0; r < R; r++) {
                    const int lr = slot * R + r;  // row within the block
                    const unsigned char* cb = sbase + (size_t)s * set_bytes + (size_t)lr * rowbytes;
                    const uint16_t* sp = (const uint16_t*)(sbase + (size_t)s * set_bytes + codes_bytes) + lr * G;
                    const uint16_t* bp = (const uint16_t*)(sbase + (size_t)s * set_bytes + codes_bytes + sb_bytes) + lr * G;
#pragma unroll
                    for (int j = 0; j < J; j++) {
                        const int g = u + j * T_row;
                        const uint4 w0 = *(const uint4*)(cb + g * 32);
                        const uint4 w1 = *(const uint4*)(cb + g * 32 + 16);
                        const uint32_t ww[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
                        int ev[8], od[8];
#pragma unroll
                        for (int i = 0; i < 8; i++) {
                            ev[i] = (int)(ww[i] & 0x0F0F0F0Fu);
                            od[i] = (int)((ww[i] >> 4) & 0x0F0F0F0Fu);
                        }
                        const float sc = __uint_as_float((uint32_t)sp[g] << 16);
                        const float bi = __uint_as_float((uint32_t)bp[g] << 16);
#pragma unroll
                        for (int m = 0; m < MT; m++) {
                            int i0 = 0, i1 = 0, i2 = 0;
#pragma unroll
                            for (int i = 0; i < 8; i++) {
                                i0 = dp4a_ss(ev[i], X[m][j][0][2 * i], i0);
                                i0 = dp4a_ss(od[i], X[m][j][0][2 * i + 1], i0);
                                i1 = dp4a_ss(ev[i], X[m][j][1][2 * i], i1);
                                i1 = dp4a_ss(od[i], X[m][j][1][2 * i + 1], i1);
                                i2 = dp4a_ss(ev[i], X[m][j][2][2 * i], i2);
                                i2 = dp4a_ss(od[i], X[m][j][2][2 * i + 1], i2);
                            }
                            const int itot = i0 * 16384 + i1 * 128 + i2;
                            const float f = (float)itot * sxp[m][j];
                            float& ac = acc[(s * R + r) * MT + m];
                            ac = fmaf(sc, f, ac);
                            ac = fmaf(bi, xq[m][j], ac);
                        }
                    }
                }
        }
        // this warp is done reading the stage: hand it back to the producer
        __syncwarp();
        if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(&empty[st])) : "memory");
        // fold the quad's partial sums; lane (b1,b0) ends up owning value index vi
        const float folded = quad_fold<V>(acc, lane);
        const int vi = V == 4 ? (lane & 3) : (V == 2 ? (lane & 1) : 0);
        const bool writer = V == 4 ? true : (V == 2 ? (lane & 2) == 0 : (lane & 3) == 0);
        const int pb = it % PR;
        if (active && writer) part[((size_t)pb * V * a.S + (size_t)vi * a.S + slot) * T4 + (u >> 2)] = folded;
        // No block-wide barrier: each warp publishes its partials on the buffer's mbarrier and
        // moves on; one warp (rotating with the block number) waits for all of them and adds the
        // T_row/4 partials of every output in a fixed order. A warp can run at most STG blocks
        // ahead of the slowest one (the weight ring throttles it), so PR >= 2*STG buffers are
        // never overwritten while they are being summed.
        __syncwarp();
        if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(&pfull[pb])) : "memory");
        if ((tid >> 5) == it % (ncons >> 5)) {
            if (!mbar_wait(&pfull[pb], (it / PR) & 1)) { if (lane == 0) atomicOr(a.status, 128u); break; }
            for (int o = lane; o < a.S * R * MT; o += 32) {
                const int sl = o / (R * MT), rm = o - sl * (R * MT);  // rm = r*MT + m
                float v0 = 0.f, v1 = 0.f;
                const float* p0 = part + ((size_t)pb * V * a.S + (size_t)rm * a.S + sl) * T4;
                for (int i = 0; i < T4; i++) v0 += p0[i];
                if (FUSE) {
                    const float* p1 = part + ((size_t)pb * V * a.S + (size_t)(R * MT + rm) * a.S + sl) * T4;
                    for (int i = 0; i < T4; i++) v1 += p1[i];
                    v0 = gelu_tanh_dev(v0) * v1;
                }
                const int r = rm / MT, m = rm - r * MT;
                const int64_t row = (int64_t)b * RB + sl * R + r;
                if (row < a.N) {
                    if (a.y_dtype == LTHN_DTYPE_BF16) ((uint16_t*)a.y)[(int64_t)m * a.N + row] = f32_to_bf16_bits(v0);
                    else ((float*)a.y)[(int64_t)m * a.N + row] = v0;
                }
            }
        }
    }
}

// ---- host side --------------------------------------------------------------------

bool dp4a_plan(int64_t N, int64_t K, int M, int fuse, int force_r, int force_s, Dp4aPlan* p) {
    if (M < 1 || M > 2 || K % 64 != 0 || N < 1) return false;
    if (fuse && M == 2) return false;
    const int G = (int)(K / 64);
    int J = 0;
    for (int cand : {1, 2}) {
        if (G % cand) continue;
        const int t = G / cand;
        if (t % 4 == 0 && t <= 352) { J = cand; break; }
    }
    if (!J) return false;
    const int T_row = G / J;
    const int sets = fuse ? 2 : 1;
    // V = sets * R * M partial sums per lane must be 1, 2 or 4
    int maxr = 4 / (sets * M);
    if (J == 2) maxr = std::min(maxr, M == 2 ? 1 : 2);
    // four rows per thread where the format allows it (fewer hand-offs per byte)
    int R = std::min(maxr, 4);
    int S = std::max(1, 288 / T_row);
    S = std::min(S, 32);
    if (force_s > 0 && force_s * T_row <= 352) S = force_s;
    if (force_r == 1 || force_r == 2 || force_r == 4) R = std::min(force_r, maxr);
    // small matrices: shrink the row block until every SM has work
    if (force_r <= 0) while (R > 1 && (N + (int64_t)S * R - 1) / ((int64_t)S * R) < 148) R >>= 1;
    if (force_s <= 0) while (S > 1 && (N + (int64_t)S * R - 1) / ((int64_t)S * R) < 148) S >>= 1;
    if ((S * R) % 2) {  // bulk copies of the scale tile need an even number of rows per block
        if (R < maxr) R *= 2; else if (S * T_row * 2 <= 352) S *= 2; else return false;
    }
    for (;;) {
        p->J = J; p->R = R; p->T_row = T_row; p->S = S;
        p->cons_threads = (S * T_row + 31) / 32 * 32;
        p->threads = p->cons_threads + 32;
        if (p->threads > 384) return false;
        p->nblocks = (int)((N + (int64_t)S * R - 1) / ((int64_t)S * R));
        p->part_bytes = (int)(((size_t)8 * sets * R * M * S * (T_row / 4) * sizeof(float) + 15) / 16 * 16);
        const size_t RB = (size_t)S * R;
        const size_t stage = sets * (RB * (K / 2) + 2 * ((RB * G * 2 + 15) / 16 * 16));
        p->smem = (size_t)p->part_bytes + 128 + 4 * stage;
        if (p->smem <= 200 * 1024) return true;
        if (R > 1 && ((S * (R / 2)) % 2 == 0)) { R /= 2; continue; }  // smaller row block, still an even row count
        return false;
    }
}

template <int J, int R, int MT, int FUSE>
static int32_t launch_dp4a_t(cudaStream_t st, const Dp4aArgs& a, const Dp4aPlan& p) {
    static int cached_dev = -1;
    static std::mutex mu;  // guards the caches below against concurrent host threads
    int dev = 0;
    LTHN_CUDA_TRY(cudaGetDevice(&dev));
    auto kern = qmv_dp4a_kernel<J, R, MT, FUSE>;
    std::unique_lock<std::mutex> lk(mu);
    if (cached_dev != dev) {
        LTHN_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
        cached_dev = dev;
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
    lk.unlock();
    int sms = 148;
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const int grid = std::min(p.nblocks, sms * occ);
    LTHN_CUDA_TRY(launch_k(kern, dim3(grid), dim3(p.threads), p.smem, st, a));
    return LTHN_OK;
}

int32_t dp4a_launch(cudaStream_t st, const QmvCall& c, const Dp4aPlan& p) {
    Dp4aArgs a{};
    a.wq[0] = c.wq; a.scales[0] = c.scales; a.biases[0] = c.biases;
    a.wq[1] = c.wq2; a.scales[1] = c.scales2; a.biases[1] = c.biases2;
    a.x = c.x; a.y = c.y; a.N = c.N; a.K = c.K; a.x_dtype = c.x_dtype; a.y_dtype = c.y_dtype;
    a.T_row = p.T_row; a.S = p.S; a.nblocks = p.nblocks; a.part_bytes = p.part_bytes;
    a.cons_threads = p.cons_threads;
    a.status = device_status_word();
    if (!a.status) return fail(LTHN_ERR_CUDA, "affine_qmv: no device status word");
    const int fuse = c.wq2 ? 1 : 0;
#define LTHN_DP4A(JJ, RR, MM, FF) \
    if (p.J == JJ && p.R == RR && c.M == MM && fuse == FF) return launch_dp4a_t<JJ, RR, MM, FF>(st, a, p);
    LTHN_DP4A(1, 4, 1, 0) LTHN_DP4A(1, 2, 1, 0) LTHN_DP4A(1, 1, 1, 0)
    LTHN_DP4A(2, 2, 1, 0) LTHN_DP4A(2, 1, 1, 0)
    LTHN_DP4A(1, 2, 2, 0) LTHN_DP4A(1, 1, 2, 0) LTHN_DP4A(2, 1, 2, 0)
    LTHN_DP4A(1, 2, 1, 1) LTHN_DP4A(1, 1, 1, 1) LTHN_DP4A(2, 1, 1, 1)
#undef LTHN_DP4A
    return fail(LTHN_ERR_INVALID, "affine_qmv: no dp4a instantiation for this plan");
}

}  // namespace lthn
