// decoder_kernels.hpp — launch wrappers of the fused decoder-step kernels.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>
#include <stddef.h>

#include <string>

namespace lthn {

constexpr int ARGMAX_BLOCKS = 64;

struct SdpaArgs {
    const float* q;            // [rows, Hq, D] f32, already normed and rotated
    const uint16_t* kcache;    // bf16, lane-major: [lanes][max_len][Hkv*D]
    const uint16_t* vcache;
    const int32_t* row_pos;    // [rows] position of the row's newest key
    const int32_t* row_lane;   // [rows] cache lane of each row
    float* out;                // [rows, Hq, D]
    float* part;               // [rows, Hq, nchunks, D+2] split-KV partials (scratch)
    int64_t lane_stride;       // elements between cache lanes
    int Hq, Hkv;
    int nchunks, chunk_len;
    float scale;
    uint16_t* cols = nullptr;  // optional bf16 split columns of the output (written by the merge stage)
    int split = 0;
    int window = 0;            // > 0: a row attends only its last `window` keys (sliding-attention block)
};

int32_t launch_geglu(cudaStream_t s, const float* g, const float* u, float* out, int64_t n);
int32_t launch_embed(cudaStream_t s, const int32_t* ids, int rows, const uint32_t* packed, const uint16_t* scales,
                     const uint16_t* biases, int hidden, int vocab, float embed_scale, float* out);
int32_t launch_rmsnorm(cudaStream_t s, const float* a, float* h, const float* w_post, const float* w_next, float* out,
                       int rows, int width, float eps, int mode, uint16_t* cols = nullptr, int split = 0);
// Tensor-parallel residual RMSNorm: the row-parallel projection before it left one partial sum
// per rank; this kernel signals "my partial is complete" to every peer, waits (bounded) for
// theirs, adds the partials in rank order straight from the peers' memory and then does the
// residual add and both norms. One kernel instead of all-reduce + norm.
struct PeerGather {
    const float* part[8];    // rank r's partial-sum buffer for this call site, as mapped on this GPU
    uint32_t* flag_out[8];   // rank r's flag array as mapped here; element [rank] is this rank's to write
    const uint32_t* flag_in; // this rank's flag array (local); element [r] is written by rank r
    uint32_t* ctr;           // local: [0] sequence number of the last finished exchange, [1] CTA arrivals
    uint32_t* status;        // device status word (bit 256: a peer's flag did not arrive in time)
    int t, rank;
    uint32_t poll_limit = 0; // polls before the wait gives up (0: the default, about a second)
};
int32_t launch_rmsnorm_gather(cudaStream_t s, const PeerGather& pg, float* h, const float* w_post, const float* w_next,
                              float* out, int rows, int width, float eps, uint16_t* cols, int split);
int32_t launch_qknorm_rope_append(cudaStream_t s, const float* qkv, const float* q_norm, const float* k_norm,
                                  const float2* rope_table, const int32_t* row_pos, const int32_t* row_lane,
                                  float* q_out, uint16_t* kcache, uint16_t* vcache, int rows, int Hq, int Hkv, int D,
                                  float eps, int64_t lane_stride, int max_len);
int32_t launch_rmsnorm_rope(cudaStream_t s, const float* x, const float* w, const int32_t* positions, float* out,
                            int rows, int heads, int D, int rotary, float eps, float rope_base, int bf16_seams);
int sdpa_chunking(int max_ctx, int D, int* chunk_len, int rows, int bundles);
int sdpa_item_chunks(int max_ctx, int D);
size_t sdpa_scratch_bytes(int rows, int Hq, int D, int nchunks);
int32_t launch_sdpa_decode(cudaStream_t s, SdpaArgs a, int rows, int D);
// Decode attention in one launch: head norms + RoPE, KV append, split-KV attention, merge.
struct SdpaFusedArgs {
    const float* qkv;          // [rows, (Hq + 2*Hkv) * D] f32 projection output
    const float* n_q;          // [D]
    const float* n_k;
    const float2* rope;        // [max_len][D/2]
    const int32_t* row_pos;
    const int32_t* row_lane;
    uint16_t* kcache;          // this block's cache
    uint16_t* vcache;
    int64_t lane_stride;
    float* out;                // [rows, Hq, D]
    float* part;               // [rows, Hq, nchunks, D+2]
    uint32_t* counters;        // [rows, Hkv], zero between launches (the kernel leaves them zero)
    int Hq, Hkv, nchunks, max_len;
    float eps, scale;
    uint16_t* cols = nullptr;  // optional bf16 split columns of the output
    int split = 0;
};
bool sdpa_fused_supported(int Hq, int Hkv, int D);
int32_t launch_sdpa_fused(cudaStream_t s, const SdpaFusedArgs& a, int rows, int D);
// Causal attention of `rows` consecutive prompt positions pos0.. of one cache lane (prefill).
struct PrefillAttnArgs {
    const float* q;          // [rows, Hq, D] f32, normed and rotated
    const uint16_t* kc;      // this lane's and layer's cache: [max_len][Hkv*D] bf16, rows 0..pos0+rows-1 valid
    const uint16_t* vc;
    uint16_t* out;           // [rows, Hq, D] bf16
    int rows, pos0, Hq, Hkv;
    float scale_log2e;       // softmax scale times log2(e)
    int window = 0;          // > 0: a row attends only its last `window` keys
};
int32_t launch_prefill_attn(cudaStream_t s, const PrefillAttnArgs& a, int D);
// ---- all decoder blocks of one token in one cooperative kernel (batch 1, one GPU) -------------
constexpr int PERSIST_SLOT_G = 44;       // groups of 64 input columns per ring slot at most
constexpr int PERSIST_SYNC_WORDS = 128;  // [0] grid-barrier arrivals, [2] abort flag, [32] finished barrier round, [64 + kv head] attention items done
struct PersistLayer {
    const uint32_t *qkv_w, *o_w, *gate_w, *up_w, *down_w;
    const uint16_t *qkv_s, *qkv_b, *o_s, *o_b, *gate_s, *gate_b, *up_s, *up_b, *down_s, *down_b;
    const float *n_input, *n_q, *n_k, *n_post_attn, *n_pre_ff, *n_post_ff;
    uint16_t *kcache, *vcache;           // this block's cache: [lanes][max_len][Hkv*D] bf16
};
struct PersistPhase { int nblk, nsl, KS, G; };  // row blocks, ring slots per row block, groups per slot, groups per row
struct PersistArgs {
    const PersistLayer* layers;          // device memory
    int nlayers;
    int H, Hq, Hkv, D, F;
    float eps, attn_scale;
    double inv_h;                        // 1 / H
    const int32_t* row_pos;              // [1] position of the token being decoded
    const int32_t* row_lane;             // [1] its cache lane
    int64_t lane_stride;
    int max_len;
    const float2* rope;                  // [max_len][D/2] (cos, sin)
    float* h0;                           // residual stream at entry (the embedding row); the two buffers alternate
    float* h1;                           //   and after 2*nlayers-1 updates the stream is in h1
    float* qkv;                          // [(Hq+2Hkv)*D]
    unsigned char* dig_att;              // digit planes of the attention output: persist_digit_bytes()
    unsigned char* dig_act;              // digit planes of the GeGLU vector: persist_digit_bytes()
    float* a;                            // [H]: o / down projection output (the last down output stays here)
    float* act;                          // [F]
    float* part;                         // [Hq][nchunks_cap][D+2] split-KV partials
    int nchunks_cap;
    uint32_t* sync;                      // PERSIST_SYNC_WORDS words, cleared by the launch wrapper
    uint32_t* status;                    // device status word
    PersistPhase ph[4];                  // q|k|v, o, gate|up, down
    int nslots, ring_off;
};
size_t persist_digit_bytes(int Hq, int D, int F);
bool persist_supported(int H, int Hq, int Hkv, int D, int F, std::string* why);
// fills ph / nslots / ring_off and the dynamic shared-memory size
int32_t persist_plan(int H, int Hq, int Hkv, int D, int F, PersistArgs* a, size_t* smem);
int32_t launch_decode_persistent(cudaStream_t s, const PersistArgs& a, size_t smem);

int32_t launch_argmax(cudaStream_t s, const float* logits, int rows, int V, float* pv, int* pi, int32_t* out_idx,
                      float* out_val, int index_offset);
int32_t launch_advance(cudaStream_t s, int32_t* row_pos, int32_t* ids, const int32_t* next, int rows);

}  // namespace lthn
