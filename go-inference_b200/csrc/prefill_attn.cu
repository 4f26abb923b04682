// prefill_attn.cu — causal attention for a chunk of prompt rows over the seq-major bf16 KV
// cache (the prefill companion of sdpa_decode_kernel), written for B200 (sm_100a).
//
//   out[r, h, :] = softmax(q[r, h, :] . K[0..pos0+r, kv(h), :]^T * scale) . V[0..pos0+r, kv(h), :]
//
// for the `rows` consecutive positions pos0 .. pos0+rows-1 of one cache lane, whose K and V rows
// (the chunk's own included) are already in the cache. It stands where the reference runs its
// batched chunked attention in prefill (engine/hip/kernels/attention/chunked.hipinc, stage 1 of
// the _batch_chunked kernels; GQA head map rocmOracleKVHeadForQuery, engine/hip/
// hip_gemma4_q4_oracle_test.go:1085-1101; arithmetic of hipReferenceSingleHeadAttentionWithScale,
// engine/hip/hip_transformer_reference.go:295-330) and follows the bf16 contract of the
// reference's Metal prefill: queries and softmax weights are rounded to bf16 for the two tensor-core
// products, scores and the output accumulate in f32.
//
// One CTA = 64 query rows of one query head, four warps of 16 rows. K and V tiles of BN keys are
// brought in with cp.async (16-byte chunks, double buffered) into shared-memory rows padded by 16
// bytes so that ldmatrix reads are conflict free; S = Q K^T and O += P V run on mma.sync m16n8k16
// (bf16 x bf16 -> f32) with the running (max, sum) softmax of one pass over the keys. The work is
// about 4*rows*keys*D flops per head against 4*keys*D bytes of K and V per 64 rows, so the kernel is
// bound by the tensor pipe, not by memory; query tiles are issued longest first.
#include "common.cuh"
#include "decoder_kernels.hpp"

#include <mutex>

namespace lthn {

__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t (&r)[4], const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void cp_async16(void* dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    return (uint32_t)f32_to_bf16_bits(lo) | ((uint32_t)f32_to_bf16_bits(hi) << 16);
}

constexpr int PA_BM = 64;       // query rows per CTA
constexpr int PA_THREADS = 128;

template <int D>
struct PaCfg {
    static constexpr int BN = D >= 256 ? 32 : 64;  // keys per tile (registers: the 16 x D f32 output tile lives in them)
    static constexpr int LD = D + 8;               // padded shared-memory row, elements
    static constexpr size_t SMEM = (size_t)(PA_BM + 4 * BN) * LD * 2;
};

template <int D>
__global__ void __launch_bounds__(PA_THREADS) prefill_attn_kernel(const PrefillAttnArgs a) {
    using C = PaCfg<D>;
    constexpr int BN = C::BN, LD = C::LD;
    constexpr int NS = BN / 8;   // score n-tiles per warp row block
    constexpr int ND = D / 8;    // output n-tiles
    extern __shared__ __align__(16) unsigned char pa_smem[];
    uint16_t* Qs = (uint16_t*)pa_smem;                 // [64][LD]
    uint16_t* Ks = Qs + PA_BM * LD;                    // [2][BN][LD]
    uint16_t* Vs = Ks + 2 * BN * LD;                   // [2][BN][LD]

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int qt = gridDim.x - 1 - blockIdx.x;  // longest tiles first
    const int m0 = qt * PA_BM, head = blockIdx.y;
    const int kvh = head / (a.Hq / a.Hkv);
    const int KR = a.Hkv * D;
    const int rows_here = min(PA_BM, a.rows - m0);
    const int kv_len = a.pos0 + m0 + rows_here;          // keys this tile may look at
    const int ntiles = (kv_len + BN - 1) / BN;
    const uint16_t* kbase = a.kc + (int64_t)kvh * D;
    const uint16_t* vbase = a.vc + (int64_t)kvh * D;

    auto load_kv = [&](int tile, int buf) {
        constexpr int CPR = D / 8;  // 16-byte chunks per row
        uint16_t* kd = Ks + buf * BN * LD;
        uint16_t* vd = Vs + buf * BN * LD;
        for (int i = tid; i < BN * CPR; i += PA_THREADS) {
            const int r = i / CPR, c = i - r * CPR;
            const int key = min(tile * BN + r, kv_len - 1);  // rows past the end are masked below; stay in bounds
            cp_async16(kd + r * LD + c * 8, kbase + (int64_t)key * KR + c * 8);
            cp_async16(vd + r * LD + c * 8, vbase + (int64_t)key * KR + c * 8);
        }
        cp_async_commit();
    };
    // sliding block: the first query row of this CTA sees keys from pos - window + 1 on; key tiles below that are skipped
    const int j0 = a.window > 0 ? max(0, a.pos0 + m0 - a.window + 1) / BN : 0;
    load_kv(j0, 0);

    // queries: f32 -> bf16 into shared memory (rows past the chunk are zero)
    for (int i = tid; i < PA_BM * (D / 4); i += PA_THREADS) {
        const int r = i / (D / 4), c = i - r * (D / 4);
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (r < rows_here) v = *(const float4*)(a.q + ((int64_t)(m0 + r) * a.Hq + head) * D + c * 4);
        *(uint2*)(Qs + r * LD + c * 4) = make_uint2(pack_bf16(v.x, v.y), pack_bf16(v.z, v.w));
    }

    float o[ND][4];
#pragma unroll
    for (int n = 0; n < ND; n++) { o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f; }
    float mrow[2] = {-INFINITY, -INFINITY}, lrow[2] = {0.f, 0.f};
    const int qpos0 = a.pos0 + m0 + warp * 16 + g;  // position of this thread's first row; the second is +8

    for (int j = j0; j < ntiles; j++) {
        const int buf = (j - j0) & 1;
        cp_async_wait<0>();
        __syncthreads();  // tile j (and, first time, the queries) visible; everyone is done with tile j-1
        if (j + 1 < ntiles) load_kv(j + 1, buf ^ 1);
        const uint16_t* kt = Ks + buf * BN * LD;
        const uint16_t* vt = Vs + buf * BN * LD;

        // ---- S = Q K^T ---------------------------------------------------------------------
        float s[NS][4];
#pragma unroll
        for (int n = 0; n < NS; n++) { s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f; }
#pragma unroll
        for (int kk = 0; kk < D / 16; kk++) {
            uint32_t qa[4];
            ldsm_x4(qa, Qs + (warp * 16 + (lane & 15)) * LD + kk * 16 + (lane >> 4) * 8);
#pragma unroll
            for (int n2 = 0; n2 < BN / 16; n2++) {
                uint32_t kb[4];
                const int mi = lane >> 3;
                ldsm_x4(kb, kt + (n2 * 16 + (mi >> 1) * 8 + (lane & 7)) * LD + kk * 16 + (mi & 1) * 8);
                mma_bf16_16816(s[2 * n2], qa[0], qa[1], qa[2], qa[3], kb[0], kb[1]);
                mma_bf16_16816(s[2 * n2 + 1], qa[0], qa[1], qa[2], qa[3], kb[2], kb[3]);
            }
        }
        // ---- mask, running softmax ---------------------------------------------------------------
        float mx[2] = {mrow[0], mrow[1]};
#pragma unroll
        for (int n = 0; n < NS; n++) {
            const int key = j * BN + n * 8 + 2 * t;
#pragma unroll
            for (int e = 0; e < 4; e++) {
                const int k = key + (e & 1), qp = qpos0 + (e >> 1) * 8;
                const float v = (k <= qp && (a.window <= 0 || k > qp - a.window)) ? s[n][e] * a.scale_log2e : -INFINITY;
                s[n][e] = v;
                mx[e >> 1] = fmaxf(mx[e >> 1], v);
            }
        }
        float alpha[2];
#pragma unroll
        for (int h = 0; h < 2; h++) {
            mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
            mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
            // a row with no visible key yet keeps max = -inf: use 0 as the reference so that exp2 stays finite
            const float mref = mx[h] == -INFINITY ? 0.f : mx[h];
            alpha[h] = exp2f(mrow[h] - mref);   // mrow = -inf -> 0
            mrow[h] = mx[h];
            mx[h] = mref;
            lrow[h] *= alpha[h];
        }
        uint32_t pfrag[NS][2];
#pragma unroll
        for (int n = 0; n < NS; n++) {
            const float p0 = exp2f(s[n][0] - mx[0]), p1 = exp2f(s[n][1] - mx[0]);
            const float p2 = exp2f(s[n][2] - mx[1]), p3 = exp2f(s[n][3] - mx[1]);
            lrow[0] += p0 + p1;
            lrow[1] += p2 + p3;
            pfrag[n][0] = pack_bf16(p0, p1);
            pfrag[n][1] = pack_bf16(p2, p3);
        }
#pragma unroll
        for (int n = 0; n < ND; n++) { o[n][0] *= alpha[0]; o[n][1] *= alpha[0]; o[n][2] *= alpha[1]; o[n][3] *= alpha[1]; }
        // ---- O += P V -------------------------------------------------------------------------------
#pragma unroll
        for (int kt16 = 0; kt16 < BN / 16; kt16++) {
            const uint32_t a0 = pfrag[2 * kt16][0], a1 = pfrag[2 * kt16][1], a2 = pfrag[2 * kt16 + 1][0], a3 = pfrag[2 * kt16 + 1][1];
#pragma unroll
            for (int d2 = 0; d2 < D / 16; d2++) {
                uint32_t vb[4];
                const int mi = lane >> 3;
                ldsm_x4_trans(vb, vt + (kt16 * 16 + (mi & 1) * 8 + (lane & 7)) * LD + d2 * 16 + (mi >> 1) * 8);
                mma_bf16_16816(o[2 * d2], a0, a1, a2, a3, vb[0], vb[1]);
                mma_bf16_16816(o[2 * d2 + 1], a0, a1, a2, a3, vb[2], vb[3]);
            }
        }
    }
    // ---- normalise and store ---------------------------------------------------------------------------
#pragma unroll
    for (int h = 0; h < 2; h++) {
        lrow[h] += __shfl_xor_sync(0xffffffffu, lrow[h], 1);
        lrow[h] += __shfl_xor_sync(0xffffffffu, lrow[h], 2);
    }
#pragma unroll
    for (int h = 0; h < 2; h++) {
        const int r = warp * 16 + g + 8 * h;
        if (r >= rows_here) continue;
        const float inv = lrow[h] > 0.f ? 1.0f / lrow[h] : 0.f;
        uint16_t* orow = a.out + ((int64_t)(m0 + r) * a.Hq + head) * D + 2 * t;
#pragma unroll
        for (int n = 0; n < ND; n++) *(uint32_t*)(orow + n * 8) = pack_bf16(o[n][2 * h] * inv, o[n][2 * h + 1] * inv);
    }
}

template <int D>
static int32_t launch_pa(cudaStream_t s, const PrefillAttnArgs& a) {
    static int attr_dev = -1;
    static std::mutex mu;
    int dev = 0;
    LTHN_CUDA_TRY(cudaGetDevice(&dev));
    {
        std::lock_guard<std::mutex> lk(mu);
        if (attr_dev != dev) {
            LTHN_CUDA_TRY(cudaFuncSetAttribute(prefill_attn_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)PaCfg<D>::SMEM));
            attr_dev = dev;
        }
    }
    dim3 grid((a.rows + PA_BM - 1) / PA_BM, a.Hq);
    prefill_attn_kernel<D><<<grid, PA_THREADS, PaCfg<D>::SMEM, s>>>(a);
    LTHN_CUDA_TRY(cudaGetLastError());
    return LTHN_OK;
}

int32_t launch_prefill_attn(cudaStream_t s, const PrefillAttnArgs& a, int D) {
    if (a.rows <= 0) return LTHN_OK;
    if (a.Hq % a.Hkv != 0) return fail(LTHN_ERR_INVALID, "prefill_attn: Hq must be a multiple of Hkv");
    if (D == 64) return launch_pa<64>(s, a);
    if (D == 128) return launch_pa<128>(s, a);
    if (D == 256) return launch_pa<256>(s, a);
    return fail(LTHN_ERR_INVALID, "prefill_attn: head_dim must be 64, 128 or 256");
}

}  // namespace lthn
