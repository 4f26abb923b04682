// sampler.cu — stochastic sampling: the reproducible sampler of the reference on the host, and
// the device half that keeps the vocabulary-wide work on the GPU.
//
// model.Sampler (model/sample.go:52-400) draws from bf16 logits: temperature, top-k, top-p, min-p,
// suppressed tokens, a repeat penalty over the generated history (sample.go:449-508), one
// splitmix64 draw per token. Its SampleCandidates form exists so that a device backend ranks the
// vocabulary itself and hands the host only a candidate window; the reference's HIP engine does
// that with a packed top-k kernel (engine/hip/kernels/sampling/topk.hipinc). Here:
//
//   device   sample_prepare_kernel   f32 logits -> bf16 (the sampler's input type), then the repeat
//            sample_penalty/suppress penalty on the history ids and -inf on suppressed ids;
//            topk_select_kernel      exact top-k of a row by (value descending, index ascending) -
//                                    the order of selectTopKDesc - by a two-level radix select on
//                                    the 16-bit keys and an index-ordered compaction, one block per
//                                    row, three passes over 0.5 MB.
//   host     Sampler                 the Go code restated line by line (same f32 operation order,
//                                    exp in f64), so a draw from the k candidates is the draw
//                                    model.Sampler.Sample makes from the whole row (sample.go:
//                                    165-175 argues the equivalence).
// Requests without a top-k cap fall back to the whole row on the host (bf16 read-back).
#include "sampler.hpp"

#include <algorithm>
#include <cmath>
#include <cstring>
#include <numeric>

namespace lthn {

// ---- device ---------------------------------------------------------------------------------
__global__ void sample_prepare_kernel(const float* __restrict__ logits, int64_t n, uint16_t* __restrict__ out) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = f32_to_bf16_bits(logits[i]);
}

// history ids: v > 0 ? v / penalty : v * penalty on the bf16 value, rounded back to bf16
// (applyRepeatPenaltyBF16Into; duplicates in the list are harmless because every write starts from
// the unpenalised logit). index_offset: first vocabulary id of this (tensor-parallel) shard.
__global__ void sample_penalty_kernel(const float* __restrict__ logits, uint16_t* __restrict__ bits, int V, int index_offset,
                                      const int32_t* __restrict__ history, int n_history, float penalty) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n_history) return;
    const int id = history[i] - index_offset;
    if (id < 0 || id >= V) return;
    float v = bf16_bits_to_f32(f32_to_bf16_bits(logits[id]));
    v = v > 0.f ? __fdiv_rn(v, penalty) : __fmul_rn(v, penalty);
    bits[id] = f32_to_bf16_bits(v);
}
// suppressed ids rank below every real token: -inf (launched after the penalty, so it wins)
__global__ void sample_suppress_kernel(uint16_t* __restrict__ bits, int V, int index_offset, const int32_t* __restrict__ suppress, int n_suppress) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n_suppress) return;
    const int id = suppress[i] - index_offset;
    if (id >= 0 && id < V) bits[id] = 0xFF80u;
}

__device__ __forceinline__ uint32_t sortable16(uint16_t b) { return (b & 0x8000u) ? (uint16_t)~b : (uint16_t)(b | 0x8000u); }

// One block of 1024 threads per row. out_idx / out_bits receive exactly k entries (k <= SAMPLE_KMAX,
// k <= V): every element above the k-th largest value and, among those equal to it, the lowest
// indices. Unordered within the k; the host orders them.
__global__ void __launch_bounds__(1024) topk_select_kernel(const uint16_t* __restrict__ bits, int V, int k, int index_offset,
                                                          int32_t* __restrict__ out_idx, uint16_t* __restrict__ out_bits) {
    __shared__ int hist[256];
    __shared__ int sel[4];        // B1, above1, B2, above2
    __shared__ int warp_gt[32], warp_eq[32];
    __shared__ int base_gt, base_eq;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint16_t* row = bits + (int64_t)blockIdx.x * V;
    int32_t* oi = out_idx + (int64_t)blockIdx.x * SAMPLE_KMAX;
    uint16_t* ob = out_bits + (int64_t)blockIdx.x * SAMPLE_KMAX;
    // pass 1: histogram of the high byte
    if (tid < 256) hist[tid] = 0;
    __syncthreads();
    for (int i = tid; i < V; i += 1024) atomicAdd(&hist[sortable16(row[i]) >> 8], 1);
    __syncthreads();
    if (tid == 0) {
        int cum = 0, b = 255;
        for (; b > 0; b--) { if (cum + hist[b] >= k) break; cum += hist[b]; }
        sel[0] = b; sel[1] = cum;
    }
    __syncthreads();
    const int B1 = sel[0], above1 = sel[1];
    // pass 2: histogram of the low byte inside that bin
    if (tid < 256) hist[tid] = 0;
    __syncthreads();
    for (int i = tid; i < V; i += 1024) {
        const uint32_t key = sortable16(row[i]);
        if ((int)(key >> 8) == B1) atomicAdd(&hist[key & 255], 1);
    }
    __syncthreads();
    if (tid == 0) {
        int cum = 0, b = 255;
        const int want = k - above1;
        for (; b > 0; b--) { if (cum + hist[b] >= want) break; cum += hist[b]; }
        sel[2] = b; sel[3] = cum;
        base_gt = 0; base_eq = 0;
    }
    __syncthreads();
    const uint32_t T = ((uint32_t)B1 << 8) | (uint32_t)sel[2];
    const int n_greater = above1 + sel[3];
    const int need_eq = k - n_greater;
    // pass 3: compaction in index order
    for (int i0 = 0; i0 < V; i0 += 1024) {
        const int i = i0 + tid;
        uint32_t key = 0;
        uint16_t b = 0;
        if (i < V) { b = row[i]; key = sortable16(b); }
        const bool gt = i < V && key > T, eq = i < V && key == T;
        const unsigned mg = __ballot_sync(0xffffffffu, gt), me = __ballot_sync(0xffffffffu, eq);
        if (lane == 0) { warp_gt[warp] = __popc(mg); warp_eq[warp] = __popc(me); }
        __syncthreads();
        int pg = base_gt, pe = base_eq;
        for (int w = 0; w < warp; w++) { pg += warp_gt[w]; pe += warp_eq[w]; }
        pg += __popc(mg & ((1u << lane) - 1u));
        pe += __popc(me & ((1u << lane) - 1u));
        if (gt) { oi[pg] = i + index_offset; ob[pg] = b; }
        if (eq && pe < need_eq) { oi[n_greater + pe] = i + index_offset; ob[n_greater + pe] = b; }
        __syncthreads();
        if (tid == 0) {
            int tg = 0, te = 0;
            for (int w = 0; w < 32; w++) { tg += warp_gt[w]; te += warp_eq[w]; }
            base_gt += tg; base_eq += te;
        }
        __syncthreads();
    }
}

int32_t sample_prepare_device(cudaStream_t s, const float* logits, int V, int index_offset, const int32_t* d_history, int n_history,
                              float penalty, const int32_t* d_suppress, int n_suppress, uint16_t* bits) {
    sample_prepare_kernel<<<(V + 255) / 256, 256, 0, s>>>(logits, V, bits);
    LTHN_CUDA_TRY(cudaGetLastError());
    if (penalty > 1.0f && n_history > 0) {
        sample_penalty_kernel<<<(n_history + 255) / 256, 256, 0, s>>>(logits, bits, V, index_offset, d_history, n_history, penalty);
        LTHN_CUDA_TRY(cudaGetLastError());
    }
    if (n_suppress > 0) {
        sample_suppress_kernel<<<(n_suppress + 255) / 256, 256, 0, s>>>(bits, V, index_offset, d_suppress, n_suppress);
        LTHN_CUDA_TRY(cudaGetLastError());
    }
    return LTHN_OK;
}

int32_t sample_topk_device(cudaStream_t s, const uint16_t* bits, int rows, int V, int k, int index_offset, int32_t* out_idx, uint16_t* out_bits) {
    if (k < 1 || k > SAMPLE_KMAX || k > V) return fail(LTHN_ERR_INVALID, "sampler: device top-k serves 1 <= k <= min(256, vocab)");
    topk_select_kernel<<<rows, 1024, 0, s>>>(bits, V, k, index_offset, out_idx, out_bits);
    LTHN_CUDA_TRY(cudaGetLastError());
    return LTHN_OK;
}

// ---- host sampler: model/sample.go restated --------------------------------------------------
float HostSampler::next() {  // splitmix64 -> uniform float32 in [0,1) (sample.go:97-104)
    state += 0x9e3779b97f4a7c15ull;
    uint64_t z = state;
    z = (z ^ (z >> 30)) * 0xbf58476d1ce4e5b9ull;
    z = (z ^ (z >> 27)) * 0x94d049bb133111ebull;
    z ^= z >> 31;
    return (float)(z >> 40) / (float)(1 << 24);
}

static bool suppressed(int32_t id, const lthn_sample_params& p) {
    for (int i = 0; i < p.n_suppress; i++) if (p.suppress[i] == id) return true;
    return false;
}
static bool rank_filter_needed(const lthn_sample_params& p, int vocab) {  // sample.go:329-337
    if (p.top_k > 0 && p.top_k < vocab) return true;
    if (p.top_p > 0 && p.top_p < 1) return true;
    return p.min_p > 0;
}
// strictly lower probability, or equal probability with a higher index (sample.go:368-376)
static bool rank_less(const std::vector<float>& probs, int a, int b) {
    if (probs[a] != probs[b]) return probs[a] < probs[b];
    return a > b;
}

// drawFromRanked (sample.go:271-327)
int32_t HostSampler::draw_from_ranked(const std::vector<int>& order, const std::vector<float>& probs, const int32_t* ids, int keep, int vocab,
                                      float sum, const lthn_sample_params& p) {
    if (p.top_p > 0 && p.top_p < 1) {
        float kept_mass = sum;
        if (keep != vocab) {
            kept_mass = 0;
            for (int i = 0; i < keep; i++) kept_mass += probs[order[i]];
        }
        float cum = 0;
        int n = 0;
        while (n < keep) {
            cum += probs[order[n]];
            n++;
            if (cum >= p.top_p * kept_mass) break;
        }
        keep = n;
    }
    if (p.min_p > 0 && keep > 0) {
        const float threshold = probs[order[0]] * p.min_p;
        int n = 0;
        while (n < keep && probs[order[n]] >= threshold) n++;
        if (n > 0) keep = n;
    }
    float ksum = 0;
    for (int i = 0; i < keep; i++) ksum += probs[order[i]];
    const float target = next() * ksum;
    float acc = 0;
    for (int i = 0; i < keep; i++) {
        acc += probs[order[i]];
        if (acc >= target) return ids ? ids[order[i]] : (int32_t)order[i];
    }
    return ids ? ids[order[keep - 1]] : (int32_t)order[keep - 1];  // floating-point fall-through
}

// sampleMapped (sample.go:141-224) with sampleTopKFirst (:230-262) and sampleMappedInVocabOrder (:379-404)
int32_t HostSampler::sample(const uint16_t* logits, const int32_t* ids, int vocab, const lthn_sample_params& p, int32_t* token) {
    auto idof = [&](int i) { return ids ? ids[i] : (int32_t)i; };
    auto top1 = [&](int32_t* out) {  // greedySuppressed / topMappedSuppressed: strict '>', first wins
        int best = -1;
        float bv = -INFINITY;
        for (int i = 0; i < vocab; i++) {
            if (suppressed(idof(i), p)) continue;
            const float v = bf16_bits_to_f32(logits[i]);
            if (v > bv) { best = i; bv = v; }
        }
        if (best < 0) return fail(LTHN_ERR_INVALID, "sampler: all tokens are suppressed");
        *out = idof(best);
        return (int32_t)LTHN_OK;
    };
    if (p.temperature <= 0 && p.min_p <= 0) return top1(token);
    if (p.top_k == 1) {
        const int32_t rc = top1(token);
        if (rc) return rc;
        next();
        return LTHN_OK;
    }
    const float temp = p.temperature <= 0 ? 1.0f : p.temperature;
    const bool rank_filter = rank_filter_needed(p, vocab);
    probs.resize(vocab);
    if (rank_filter && p.top_k > 0 && p.top_k < vocab) {
        // top-k first: rank on the temperature-scaled logits, exp only the survivors
        int allowed = 0;
        for (int i = 0; i < vocab; i++) {
            if (suppressed(idof(i), p)) { probs[i] = -INFINITY; continue; }
            probs[i] = bf16_bits_to_f32(logits[i]) / temp;
            allowed++;
        }
        if (allowed == 0) return fail(LTHN_ERR_INVALID, "sampler: all tokens are suppressed");
        const int keep = std::min(p.top_k, vocab);
        order.resize(vocab);
        std::iota(order.begin(), order.end(), 0);
        // the first `keep` of a stable descending sort = the `keep` highest under rank_less, best first
        std::partial_sort(order.begin(), order.begin() + keep, order.end(), [&](int a, int b) { return rank_less(probs, b, a); });
        order.resize(keep);
        const float max_l = probs[order[0]];
        for (int i = 0; i < keep; i++) probs[order[i]] = (float)std::exp((double)(probs[order[i]] - max_l));
        *token = draw_from_ranked(order, probs, ids, keep, vocab, 0, p);
        return LTHN_OK;
    }
    float max_l = -INFINITY;
    int allowed = 0;
    for (int i = 0; i < vocab; i++) {
        if (suppressed(idof(i), p)) continue;
        const float v = bf16_bits_to_f32(logits[i]) / temp;
        allowed++;
        if (v > max_l) max_l = v;
    }
    if (allowed == 0) return fail(LTHN_ERR_INVALID, "sampler: all tokens are suppressed");
    float sum = 0;
    for (int i = 0; i < vocab; i++) {
        if (suppressed(idof(i), p)) { probs[i] = 0; continue; }
        const float v = bf16_bits_to_f32(logits[i]) / temp;
        const float e = (float)std::exp((double)(v - max_l));
        probs[i] = e;
        sum += e;
    }
    if (!rank_filter) {
        if (sum == 0) return fail(LTHN_ERR_INVALID, "sampler: empty sampled distribution");
        const float target = next() * sum;
        float acc = 0;
        for (int i = 0; i < vocab; i++) {
            acc += probs[i];
            if (acc >= target) { *token = idof(i); return LTHN_OK; }
        }
        *token = idof(vocab - 1);
        return LTHN_OK;
    }
    order.resize(vocab);
    std::iota(order.begin(), order.end(), 0);
    std::stable_sort(order.begin(), order.end(), [&](int a, int b) { return probs[a] > probs[b]; });
    *token = draw_from_ranked(order, probs, ids, vocab, vocab, sum, p);
    return LTHN_OK;
}

}  // namespace lthn

using namespace lthn;

extern "C" {

int32_t lthn_sampler_create(uint64_t seed, void** sampler) {
    clear_error();
    LTHN_REQUIRE(sampler != nullptr, "lthn_sampler_create: NULL argument");
    HostSampler* s = new HostSampler();
    s->state = seed;
    *sampler = s;
    return LTHN_OK;
}
int32_t lthn_sampler_destroy(void* sampler) {
    clear_error();
    delete (HostSampler*)sampler;
    return LTHN_OK;
}
float lthn_sampler_draw(void* sampler) { return sampler ? ((HostSampler*)sampler)->next() : 0.0f; }

static int32_t check_params(const lthn_sample_params* p) {
    LTHN_REQUIRE(p != nullptr, "sampler: params is NULL");
    LTHN_REQUIRE(p->n_suppress >= 0 && (p->n_suppress == 0 || p->suppress != nullptr), "sampler: bad suppress list");
    return LTHN_OK;
}

int32_t lthn_sampler_sample(void* sampler, const uint16_t* logits_bf16, int32_t vocab, const lthn_sample_params* params, int32_t* token) {
    clear_error();
    LTHN_REQUIRE(sampler && logits_bf16 && token && vocab > 0, "lthn_sampler_sample: bad arguments");
    int32_t rc = check_params(params);
    if (rc) return rc;
    return ((HostSampler*)sampler)->sample(logits_bf16, nullptr, vocab, *params, token);
}

int32_t lthn_sampler_sample_candidates(void* sampler, const uint16_t* logits_bf16, const int32_t* ids, int32_t n,
                                       const lthn_sample_params* params, int32_t* token) {
    clear_error();
    LTHN_REQUIRE(sampler && logits_bf16 && ids && token, "lthn_sampler_sample_candidates: NULL argument");
    LTHN_REQUIRE(n > 0, "lthn_sampler_sample_candidates: empty candidates");
    int32_t rc = check_params(params);
    if (rc) return rc;
    return ((HostSampler*)sampler)->sample(logits_bf16, ids, n, *params, token);
}

int32_t lthn_topk_candidates(void* stream, const float* logits, int32_t rows, int32_t vocab, int32_t k, uint16_t* scratch_bf16,
                             int32_t* out_ids, uint16_t* out_bf16) {
    clear_error();
    if (rows == 0) return LTHN_OK;
    LTHN_REQUIRE(logits && scratch_bf16 && out_ids && out_bf16 && rows > 0 && vocab > 0, "lthn_topk_candidates: bad arguments");
    cudaStream_t s = (cudaStream_t)stream;
    sample_prepare_kernel<<<(unsigned)(((int64_t)rows * vocab + 255) / 256), 256, 0, s>>>(logits, (int64_t)rows * vocab, scratch_bf16);
    LTHN_CUDA_TRY(cudaGetLastError());
    return sample_topk_device(s, scratch_bf16, rows, vocab, k, 0, out_ids, out_bf16);
}

}  // extern "C"
