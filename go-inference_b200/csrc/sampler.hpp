// sampler.hpp — internal interface of the sampler (sampler.cu) for the engine.
#pragma once
#include "common.cuh"

#include <vector>

namespace lthn {

constexpr int SAMPLE_KMAX = 256;  // candidates the device top-k returns per row

// model.Sampler restated (model/sample.go): splitmix64 state advanced once per stochastic draw,
// scratch grown once and reused. Not for concurrent use, like the original.
struct HostSampler {
    uint64_t state = 0;
    std::vector<float> probs;
    std::vector<int> order;
    float next();
    // logits: n bf16 values; ids: NULL (token = index) or the n candidate ids the values belong to
    int32_t sample(const uint16_t* logits, const int32_t* ids, int n, const lthn_sample_params& p, int32_t* token);
    int32_t draw_from_ranked(const std::vector<int>& order, const std::vector<float>& probs, const int32_t* ids, int keep, int vocab,
                             float sum, const lthn_sample_params& p);
};

// bits[V] = bf16(logits[V]) with the repeat penalty applied to the history ids and -inf on the
// suppressed ids (both lists in device memory, ids are vocabulary ids; index_offset = first id of
// this vocabulary shard).
int32_t sample_prepare_device(cudaStream_t s, const float* logits, int V, int index_offset, const int32_t* d_history, int n_history,
                              float penalty, const int32_t* d_suppress, int n_suppress, uint16_t* bits);
// exact top-k per row (unordered within the k): out_idx / out_bits [rows][SAMPLE_KMAX]
int32_t sample_topk_device(cudaStream_t s, const uint16_t* bits, int rows, int V, int k, int index_offset, int32_t* out_idx, uint16_t* out_bits);

}  // namespace lthn
