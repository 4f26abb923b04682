// attn_item.cuh — one (kv head, key chunk) item of decode attention on a group of 128 threads,
// shared by the stand-alone fused attention kernel (decoder_kernels.cu) and the one-kernel decode
// step (decode_persistent.cu).
#pragma once
#include "common.cuh"

namespace lthn {

struct AttnItemArgs {
    const float* qkv;        // this row's projection output: Hq q heads, Hkv k heads, Hkv v heads of D values
    const float* n_q;        // [D] per-head norm weights
    const float* n_k;
    const float2* rope;      // [max_len][D/2] (cos, sin)
    uint16_t* kc;            // this row's cache lane of this block: [max_len][Hkv*D] bf16
    uint16_t* vc;
    float* part;             // this row's split-KV partials: [Hq][nchunks_cap][D+2]
    uint32_t* counter;       // this row's [Hkv] counters of finished items (zero between uses)
    int Hq, Hkv, nchunks_cap, max_len;
    float eps, scale;
};

// The arithmetic of sdpa_decode_kernel / sdpa_merge_kernel (decoder_kernels.cu) with the per-head
// RMSNorm + RoPE of q (and of the new key), the KV append and the digit planes of the output (the
// o projection's activations) folded in. Every global load of an item is issued before anything
// is computed: one memory round trip per item.
template <int D, int GQ>
struct alignas(16) AttnItemSmem {
    float red[4][GQ][D + 2];
    float q[GQ][D];
    uint16_t knew[D], vnew[D];
    float smax[GQ][4], ssum[GQ][4];
    double sh[4][GQ + 1];
    uint32_t last;
};

template <int D, int GQ, typename Bar, typename Emit>
__device__ __forceinline__ void attn_item(const AttnItemArgs& a, AttnItemSmem<D, GQ>& s, Bar bar, Emit emit, int kvh, int chunk, int used, int pos) {
    constexpr int E = D / 8, V8 = E / 8, NIT = 512 / D > 0 ? 512 / D : 1, CH = 16 * NIT, half = D / 2;
    const int gt = threadIdx.x & 127, lane = gt & 31, warp = gt >> 5;
    const int l8 = lane & 7, pg = warp * 4 + (lane >> 3);
    const int ctx = pos + 1, p0 = chunk * CH, KR = a.Hkv * D, qh0 = kvh * GQ;
    uint16_t* kbase = a.kc + (int64_t)kvh * D;
    uint16_t* vbase = a.vc + (int64_t)kvh * D;
    const bool has_new = pos >= p0 && pos < p0 + CH;  // this chunk holds the token being decoded
    const bool pair = gt < half;                      // thread owns the rotation pair (gt, gt + half)

    // ---- every load of the item goes out first ---------------------------------------------------
    uint4 kreg[NIT][V8], vreg[NIT][V8];
    bool valid[NIT];
#pragma unroll
    for (int i = 0; i < NIT; i++) {
        const int p = p0 + pg + 16 * i;
        valid[i] = p < ctx;
        const int64_t off = (int64_t)((valid[i] && p != pos) ? p : p0) * KR;  // the new token's row comes from shared memory
#pragma unroll
        for (int v = 0; v < V8; v++) {
            kreg[i][v] = __ldcg((const uint4*)(kbase + off + (v * 8 + l8) * 8));
            vreg[i][v] = __ldcg((const uint4*)(vbase + off + (v * 8 + l8) * 8));
        }
    }
    float x0[GQ + 1], x1[GQ + 1], w0[2], w1[2], vn0 = 0.f, vn1 = 0.f;
    float2 cs = make_float2(1.f, 0.f);
#pragma unroll
    for (int h = 0; h <= GQ; h++) {
        x0[h] = 0.f; x1[h] = 0.f;
        if (pair && (h < GQ || has_new)) {
            const float* src = a.qkv + (int64_t)(h < GQ ? qh0 + h : a.Hq + kvh) * D;
            x0[h] = __ldcg(src + gt);
            x1[h] = __ldcg(src + gt + half);
        }
    }
    w0[0] = w0[1] = w1[0] = w1[1] = 0.f;
    if (pair) {
        cs = __ldg(a.rope + (int64_t)min(pos, a.max_len - 1) * half + gt);
        w0[0] = __ldg(a.n_q + gt); w1[0] = __ldg(a.n_q + gt + half);
        if (has_new) {
            w0[1] = __ldg(a.n_k + gt); w1[1] = __ldg(a.n_k + gt + half);
            const float* src = a.qkv + (int64_t)(a.Hq + a.Hkv + kvh) * D;
            vn0 = __ldcg(src + gt); vn1 = __ldcg(src + gt + half);
        }
    }
    // ---- head norms + RoPE ---------------------------------------------------------------------------
    double ss[GQ + 1];
#pragma unroll
    for (int h = 0; h <= GQ; h++) {
        ss[h] = (double)__fmul_rn(x0[h], x0[h]) + (double)__fmul_rn(x1[h], x1[h]);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) ss[h] += __shfl_xor_sync(0xffffffffu, ss[h], o);
    }
    bar();  // the previous item's readers of this scratch are done
    if (lane == 0)
#pragma unroll
        for (int h = 0; h <= GQ; h++) s.sh[warp][h] = ss[h];
    bar();
#pragma unroll
    for (int h = 0; h <= GQ; h++) {
        if (h == GQ && !has_new) continue;
        const double tsum = s.sh[0][h] + s.sh[1][h] + s.sh[2][h] + s.sh[3][h];
        const FastDiv k = fast_div_by(fast_rms(tsum, 1.0 / (double)D, a.eps));
        if (pair) {
            const float n0 = __fmul_rn(fast_div(x0[h], k), w0[h < GQ ? 0 : 1]);
            const float n1 = __fmul_rn(fast_div(x1[h], k), w1[h < GQ ? 0 : 1]);
            const float r0 = __fsub_rn(__fmul_rn(n0, cs.x), __fmul_rn(n1, cs.y));
            const float r1 = __fadd_rn(__fmul_rn(n0, cs.y), __fmul_rn(n1, cs.x));
            if (h < GQ) {
                s.q[h][gt] = r0 * a.scale;
                s.q[h][gt + half] = r1 * a.scale;
            } else {
                const uint16_t b0 = f32_to_bf16_bits(r0), b1 = f32_to_bf16_bits(r1);
                s.knew[gt] = b0; s.knew[gt + half] = b1;
                uint16_t* dst = kbase + (int64_t)pos * KR;
                dst[gt] = b0; dst[gt + half] = b1;
            }
        }
    }
    if (has_new && pair) {
        const uint16_t b0 = f32_to_bf16_bits(vn0), b1 = f32_to_bf16_bits(vn1);
        s.vnew[gt] = b0; s.vnew[gt + half] = b1;
        uint16_t* dst = vbase + (int64_t)pos * KR;
        dst[gt] = b0; dst[gt + half] = b1;
    }
    bar();  // q and the new row are in shared memory
    if (has_new) {
#pragma unroll
        for (int i = 0; i < NIT; i++)
            if (p0 + pg + 16 * i == pos) {
#pragma unroll
                for (int v = 0; v < V8; v++) {
                    kreg[i][v] = *(const uint4*)(&s.knew[(v * 8 + l8) * 8]);
                    vreg[i][v] = *(const uint4*)(&s.vnew[(v * 8 + l8) * 8]);
                }
            }
    }
    float q[GQ][E];
#pragma unroll
    for (int h = 0; h < GQ; h++)
#pragma unroll
        for (int v = 0; v < V8; v++) {
            const float4 qa = *(const float4*)(&s.q[h][(v * 8 + l8) * 8]);
            const float4 qb = *(const float4*)(&s.q[h][(v * 8 + l8) * 8 + 4]);
            q[h][v * 8 + 0] = qa.x; q[h][v * 8 + 1] = qa.y; q[h][v * 8 + 2] = qa.z; q[h][v * 8 + 3] = qa.w;
            q[h][v * 8 + 4] = qb.x; q[h][v * 8 + 5] = qb.y; q[h][v * 8 + 6] = qb.z; q[h][v * 8 + 7] = qb.w;
        }
    // ---- scores ----------------------------------------------------------------------------------------
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
        if (lane == 0) s.smax[h][warp] = m;
    }
    bar();
    float cmax[GQ];
#pragma unroll
    for (int h = 0; h < GQ; h++) cmax[h] = fmaxf(fmaxf(s.smax[h][0], s.smax[h][1]), fmaxf(s.smax[h][2], s.smax[h][3]));
    // ---- weights and weighted values ---------------------------------------------------------------------
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
        if (lane == 0) s.ssum[h][warp] = l;
        if (lane < 8) {
#pragma unroll
            for (int v = 0; v < V8; v++)
#pragma unroll
                for (int e = 0; e < 8; e++) s.red[warp][h][(v * 8 + l8) * 8 + e] = acc[h][v * 8 + e];
        }
    }
    bar();
    // (every thread of the group is past its reads of s.q: the query went to registers before the barriers above)
    for (int idx = gt; idx < GQ * D; idx += 128) {
        const int h = idx / D, d = idx - h * D;
        const float v = s.red[0][h][d] + s.red[1][h][d] + s.red[2][h][d] + s.red[3][h][d];
        const float l = s.ssum[h][0] + s.ssum[h][1] + s.ssum[h][2] + s.ssum[h][3];
        if (used == 1) {
            s.q[h][d] = fast_div(v, fast_div_by(l));
        } else {
            float* pa = a.part + ((int64_t)(qh0 + h) * a.nchunks_cap + chunk) * (D + 2);
            pa[d] = v;
            if (d == 0) { pa[D] = cmax[h]; pa[D + 1] = l; }
        }
    }
    bool done = used == 1;
    if (!done) {
    // ---- the last item of this kv head to finish merges the head's chunk partials ----------------
    __threadfence();
    bar();
    if (gt == 0) {
        const uint32_t n = atomicAdd(a.counter + kvh, 1u);
        s.last = (n == (uint32_t)used - 1u) ? 1u : 0u;
        if (s.last) { a.counter[kvh] = 0u; __threadfence(); }
    }
    bar();
    done = s.last != 0;
    if (done) {
    // One pass over the chunks for both heads (the loads of MB chunks per warp are issued together);
    // warp w takes chunks w, w+4, ..., lane D/32 consecutive dimensions.
    constexpr int DL = D / 32, MB = 4;
    float m[GQ], l[GQ], macc[GQ][DL];
#pragma unroll
    for (int h = 0; h < GQ; h++) {
        m[h] = -INFINITY; l[h] = 0.f;
#pragma unroll
        for (int i = 0; i < DL; i++) macc[h][i] = 0.f;
    }
    for (int c0 = warp; c0 < used; c0 += 4 * MB) {
        float cm[GQ][MB], cl[GQ][MB];
        float2 cv[GQ][MB][DL / 2];
#pragma unroll
        for (int h = 0; h < GQ; h++)
#pragma unroll
            for (int b = 0; b < MB; b++) {
                const int c = c0 + 4 * b;
                const bool live = c < used;
                const float* p = a.part + ((int64_t)(qh0 + h) * a.nchunks_cap + (live ? c : c0)) * (D + 2);
                cm[h][b] = live ? __ldcg(p + D) : -INFINITY;
                cl[h][b] = live ? __ldcg(p + D + 1) : 0.f;
                const float2* src = (const float2*)(p + lane * DL);
#pragma unroll
                for (int i = 0; i < DL / 2; i++) cv[h][b][i] = __ldcg(src + i);
            }
#pragma unroll
        for (int h = 0; h < GQ; h++) {
            float bm = m[h];
#pragma unroll
            for (int b = 0; b < MB; b++) bm = fmaxf(bm, cm[h][b]);
            if (bm == -INFINITY) continue;
            const float rescale = __expf(m[h] - bm);
            l[h] *= rescale;
#pragma unroll
            for (int i = 0; i < DL; i++) macc[h][i] *= rescale;
#pragma unroll
            for (int b = 0; b < MB; b++) {
                const float w = __expf(cm[h][b] - bm);
                l[h] = fmaf(cl[h][b], w, l[h]);
#pragma unroll
                for (int i = 0; i < DL / 2; i++) {
                    macc[h][2 * i] = fmaf(cv[h][b][i].x, w, macc[h][2 * i]);
                    macc[h][2 * i + 1] = fmaf(cv[h][b][i].y, w, macc[h][2 * i + 1]);
                }
            }
            m[h] = bm;
        }
    }
#pragma unroll
    for (int h = 0; h < GQ; h++) {
        if (lane == 0) { s.smax[h][warp] = m[h]; s.ssum[h][warp] = l[h]; }
#pragma unroll
        for (int i = 0; i < DL; i++) s.red[warp][h][lane * DL + i] = macc[h][i];
    }
    bar();
    for (int idx = gt; idx < GQ * D; idx += 128) {
        const int h = idx / D, d = idx - h * D;
        const float gm = fmaxf(fmaxf(s.smax[h][0], s.smax[h][1]), fmaxf(s.smax[h][2], s.smax[h][3]));
        float num = 0.f, den = 0.f;
#pragma unroll
        for (int w = 0; w < 4; w++) {
            const float e = __expf(s.smax[h][w] - gm);
            num = fmaf(s.red[w][h][d], e, num);
            den = fmaf(s.ssum[h][w], e, den);
        }
        s.q[h][d] = fast_div(num, fast_div_by(den));
    }
    }
    }
    if (!done) return;
    bar();
    emit(s, qh0);
}


}  // namespace lthn
