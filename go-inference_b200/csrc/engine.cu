// engine.cu — the decoder engine behind the C ABI: resident 4-bit weights, the
// seq-major bf16 KV cache, retained sessions and multi-lane batched decode.
//
// It mirrors what a go-inference engine package supplies to the shared adapters:
//   Model    -> engine.TokenModel (engine/model.go:25-31): weights stay resident,
//               OpenEngineSession hands out a Session over a free KV lane.
//   Session  -> engine.Session (engine/session.go:40-61): PrefillTokens / AppendTokens /
//               Pos / GenerateFromCacheEach (greedy) plus logits read-out for host-side
//               sampling.
//   LaneSet  -> inference.LaneSet (batch_step.go:97-119): K lanes with their own KV and
//               position advanced by ONE batched forward per Step.
// The forward follows the reference's layer order (engine/hip/hip_gemma4_q4_layer.go:
// 1441-2067; CPU oracle hip_gemma4_q4_oracle_test.go:873-961) for the gemma3 block:
//   norm -> q|k|v projection -> per-head norm + RoPE + KV append -> attention -> o proj
//   -> post-norm + residual + pre-FF norm -> gate|up + GeGLU -> down -> post-norm +
//   residual (+ the next layer's input norm), final norm, tied lm_head, greedy argmax.
// Activations are f32 between kernels; K and V are rounded to bf16 when appended.
//
// Tensor parallelism (no counterpart in the reference, which is single-device):
// q/k/v/gate/up are sharded by output rows (heads), o/down by input columns in whole
// 64-wide groups, the KV cache by kv head; each rank's partial o/down output is summed
// with one all-reduce (NCCL, loaded at run time) per projection.
#include "common.cuh"
#include "decoder_kernels.hpp"
#include "qmv.hpp"
#include "sampler.hpp"

#include <dlfcn.h>

#include <algorithm>
#include <chrono>
#include <cmath>
#include <cstring>
#include <memory>
#include <mutex>
#include <string>
#include <vector>

namespace lthn {

// ---- NCCL, bound at run time so the library loads without it --------------------------
struct UniqueId { char internal[128]; };
struct NcclApi {
    void* lib = nullptr;
    int (*GetUniqueId)(void*) = nullptr;
    int (*CommInitRank)(void**, int, UniqueId /* ncclUniqueId, passed by value */, int) = nullptr;
    int (*CommDestroy)(void*) = nullptr;
    int (*AllReduce)(const void*, void*, size_t, int, int, void*, cudaStream_t) = nullptr;
    int (*AllGather)(const void*, void*, size_t, int, void*, cudaStream_t) = nullptr;
    const char* (*GetErrorString)(int) = nullptr;
};
static NcclApi g_nccl;
static std::mutex g_nccl_mu;

static int32_t nccl_load() {
    std::lock_guard<std::mutex> lk(g_nccl_mu);
    if (g_nccl.lib) return LTHN_OK;
    const char* names[] = {getenv("LTHN_CUDA_NCCL_LIB"), "libnccl.so.2", "libnccl.so"};
    void* h = nullptr;
    for (const char* n : names) {
        if (!n || !*n) continue;
        h = dlopen(n, RTLD_NOW | RTLD_GLOBAL);
        if (h) break;
    }
    if (!h) return fail(LTHN_ERR_UNAVAILABLE, "NCCL not found (set LTHN_CUDA_NCCL_LIB to libnccl.so.2)");
    g_nccl.GetUniqueId = (decltype(g_nccl.GetUniqueId))dlsym(h, "ncclGetUniqueId");
    g_nccl.CommInitRank = (decltype(g_nccl.CommInitRank))dlsym(h, "ncclCommInitRank");
    g_nccl.CommDestroy = (decltype(g_nccl.CommDestroy))dlsym(h, "ncclCommDestroy");
    g_nccl.AllReduce = (decltype(g_nccl.AllReduce))dlsym(h, "ncclAllReduce");
    g_nccl.AllGather = (decltype(g_nccl.AllGather))dlsym(h, "ncclAllGather");
    g_nccl.GetErrorString = (decltype(g_nccl.GetErrorString))dlsym(h, "ncclGetErrorString");
    if (!g_nccl.GetUniqueId || !g_nccl.CommInitRank || !g_nccl.AllReduce || !g_nccl.AllGather || !g_nccl.CommDestroy) {
        dlclose(h);
        return fail(LTHN_ERR_UNAVAILABLE, "NCCL library lacks a required symbol");
    }
    g_nccl.lib = h;
    return LTHN_OK;
}
static int32_t nccl_check(int rc, const char* what) {
    if (rc == 0) return LTHN_OK;
    return fail(LTHN_ERR_CUDA, std::string(what) + ": NCCL error " + (g_nccl.GetErrorString ? g_nccl.GetErrorString(rc) : "?"));
}
enum { kNcclFloat32 = 7, kNcclSum = 0 };

// ---- model --------------------------------------------------------------------------
struct Linear {
    uint32_t* wq = nullptr; uint16_t* s = nullptr; uint16_t* b = nullptr;
    int64_t N = 0, K = 0;  // local (sharded) shape
    int bits = 4;          // 8 for an MLP projection of a mixed-precision pack
};
enum { ROLE_Q = 0, ROLE_K, ROLE_V, ROLE_O, ROLE_GATE, ROLE_UP, ROLE_DOWN, ROLE_COUNT };
// phases of a decode step as the tracer reports them
enum { PH_EMBED = 0, PH_ATTN, PH_MLP, PH_EXCHANGE, PH_BLOCKS, PH_HEAD, PH_COUNT };
static const char* const kPhaseName[PH_COUNT] = {"embedding", "attention: q|k|v, norms + rope, sdpa, o", "mlp: norms, gate|up, down",
                                                 "tensor-parallel exchange", "decoder blocks (one kernel)", "head: final norm, lm_head, argmax"};
enum { NORM_INPUT = 0, NORM_POST_ATTN, NORM_PRE_FF, NORM_POST_FF, NORM_Q, NORM_K, NORM_COUNT };

struct Layer {
    Linear qkv, o, gate, up, down;
    float* norm[NORM_COUNT] = {};
    bool have[ROLE_COUNT] = {};
};

constexpr int kMaxRows = 32;  // rows per forward (the batched matvec serves up to 32)
// Prompt rows per prefill chunk. The reference prefills in 512-token chunks
// (decode/generate/generate.go:147-150); a chunk here is four times that, because a 512-row
// projection is only 2 x N/128 tiles for 148 SMs and 512 rows x 8 heads of attention only 64 CTAs.
constexpr int kPrefillRows = 2048;

// lm_head (value, index) gather over peer memory (see tp_pair_gather_kernel)
struct PairGather {
    float* pairs_out[8];        // rank r's pair area as mapped here: [t][kMaxRows][2] floats
    const float* pairs_in;      // this rank's pair area (local)
    uint32_t* flag_out[8];
    const uint32_t* flag_in;
    uint32_t* ctr;
    uint32_t* status;
    int t, rank, max_rows;
};


struct Model {
    lthn_model_config c{};
    int Hq_l = 0, Hkv_l = 0, QR_l = 0, KR_l = 0, F_l = 0, V_l = 0, v0 = 0;
    std::vector<Layer> layers;
    Linear embed;       // full table (embedding lookup)
    Linear head;        // lm_head shard: rows [v0, v0+V_l) of the tied table (aliases embed)
    bool have_embed = false;
    float* final_norm = nullptr;
    float2* rope = nullptr;
    float2* rope_local = nullptr;  // sliding-attention blocks rotate with rope_local_base
    uint16_t *kcache = nullptr, *vcache = nullptr;
    int64_t lane_stride = 0, layer_stride = 0;
    std::vector<char> lane_used;
    bool finalized = false;
    void* comm = nullptr;
    cudaStream_t stream = nullptr;
    // workspace for up to kMaxRows rows
    int32_t *d_ids = nullptr, *d_pos = nullptr, *d_lane = nullptr, *d_next = nullptr;
    float *h = nullptr, *h2 = nullptr, *xn = nullptr, *qkv = nullptr, *q = nullptr, *att = nullptr, *a = nullptr, *act = nullptr;
    uint16_t *xn_cols = nullptr, *att_cols = nullptr;  // bf16 split columns of xn / att for the tensor-core matvec
    float *logits = nullptr, *amax_v = nullptr, *sdpa_part = nullptr, *best_v = nullptr, *gather = nullptr;
    int* amax_i = nullptr;
    size_t sdpa_part_bytes = 0;
    int32_t* h_pinned = nullptr;  // pinned staging for ids / positions / tokens
    uint64_t weight_bytes = 0;
    // one captured decode step per row count (all rows produce a token); positions, ids and
    // lanes are read from device buffers, so the same graph serves every step
    cudaGraphExec_t step_graph[kMaxRows + 1] = {};
    bool step_warm[kMaxRows + 1] = {};
    bool graphs_off = false;
    std::mutex mu;
    std::vector<void*> allocs;
    // tensor-parallel exchange over peer memory (see xchg_setup): one IPC-shared allocation per rank
    // holding the flag array and one partial-sum buffer per call site (attention output, FFN output)
    void* x_base = nullptr;
    void* x_peer[8] = {};
    uint32_t* x_ctr = nullptr;
    PeerGather pg[2] = {};
    PairGather pairg = {};
    float* x_part[2] = {};      // this rank's own slot of each call site (pull mode)
    float* x_site[2] = {};      // slot 0 of each call site in this rank's region (push mode reads all t slots)
    float* x_push[2][8] = {};   // this rank's slot of each call site in every rank's region
    int64_t x_stride = 0;       // floats between slots
    PeerWait* d_pw = nullptr;       // device copy of the exchange's wait descriptor
    float** d_push[2] = {};         // device arrays of x_push[site]
    bool site_fused[2] = {};    // tensor parallel: the site's norm runs inside the consuming matvec (push mode)
    bool xchg_ready = false;
    bool fuse_norm = false;  // batch 1-2: norms run inside the matvec that consumes them
    // mixed precision: some MLP projections hold 8-bit codes; their gate and up run as separate matvecs into g8 / u8
    bool mixed = false;
    bool pair8_ok = false;  // an 8-bit gate/up pair of this shape runs as one fused matvec for one and two rows
    float *g8 = nullptr, *u8 = nullptr;
    uint16_t* x8 = nullptr;  // bf16 activations of a 3..32-row step entering an 8-bit linear
    // engine.DecodePhaseTracer: while on, one-row decode steps run kernel by kernel with an event between phases
    struct PhaseTrace {
        bool on = false;
        std::vector<cudaEvent_t> ev;
        std::vector<int> ends;      // the phase that ends at event i (-1: start of the step)
        size_t used = 0;
        double phase_us[PH_COUNT] = {};
        double gpu_us = 0;
        int tokens = 0;
        std::chrono::steady_clock::time_point t0;
    } trace;
    // batch 1 on one GPU: every decoder block of a token in one cooperative kernel (decode_persistent.cu)
    bool attn_fused = false;       // one or two rows: norms + rope + append + attention + merge in one launch
    uint32_t* att_ctr = nullptr;  // its per-(row, kv head) counters
    bool persist_ok = false;
    PersistArgs pk{};
    size_t pk_smem = 0;
    // The logits buffer is shared by every session and lane set of the model: each forward that
    // computes logits takes the next serial number, and a lane remembers the serial of its own
    // last forward, so a read-out can tell whether the buffer still holds that lane's row.
    uint64_t logits_serial = 0;
    // prefill on the tensor cores (prompts longer than kMaxRows): chunk workspace for kPrefillRows rows
    bool prefill_tc = false;
    int prefill_rows = 0;  // rows per chunk (kPrefillRows unless LTHN_CUDA_PREFILL_CHUNK asks for fewer)
    int32_t *p_ids = nullptr, *p_pos = nullptr, *p_lane = nullptr, *p_pinned = nullptr;
    float *p_h = nullptr, *p_qkv = nullptr, *p_q = nullptr, *p_a = nullptr, *p_xnf = nullptr;
    uint16_t *p_xn = nullptr, *p_att = nullptr, *p_act = nullptr;
    // sampling workspace (first sampled call): bf16 row, candidate window, id lists
    uint16_t *s_bits = nullptr, *s_cbits = nullptr;
    int32_t *s_cidx = nullptr, *s_lists = nullptr;
    float* s_gather = nullptr;
    std::vector<uint16_t> s_host_bits;
};

template <typename T>
static int32_t dalloc(Model* m, T** p, size_t n) {
    void* q = nullptr;
    LTHN_CUDA_TRY(cudaMalloc(&q, std::max<size_t>(n * sizeof(T), 256)));
    m->allocs.push_back(q);
    *p = (T*)q;
    return LTHN_OK;
}

static int32_t linear_alloc(Model* m, Linear* l, int64_t N, int64_t K) {
    l->N = N; l->K = K;
    int32_t rc;
    if ((rc = dalloc(m, &l->wq, (size_t)N * K / 8))) return rc;
    if ((rc = dalloc(m, &l->s, (size_t)N * K / 64))) return rc;
    if ((rc = dalloc(m, &l->b, (size_t)N * K / 64))) return rc;
    m->weight_bytes += (uint64_t)N * K * 9 / 16;
    return LTHN_OK;
}

static int32_t model_validate(const lthn_model_config& c) {
    LTHN_REQUIRE(c.layers > 0 && c.hidden > 0 && c.q_heads > 0 && c.kv_heads > 0 && c.head_dim > 0 && c.ffn > 0 && c.vocab > 0,
                 "model: dimensions must be positive");
    LTHN_REQUIRE(c.group_size == 64 && c.bits == 4, "model: the decoder serves 4-bit, group-64 affine weights");
    LTHN_REQUIRE(c.q_heads % c.kv_heads == 0, "model: q_heads must be a multiple of kv_heads");
    LTHN_REQUIRE(c.head_dim == 64 || c.head_dim == 128 || c.head_dim == 256 || c.head_dim == 512, "model: head_dim must be 64, 128, 256 or 512");
    LTHN_REQUIRE(c.hidden % 64 == 0 && c.ffn % 64 == 0, "model: hidden and ffn must be multiples of the group size");
    LTHN_REQUIRE(c.max_len > 0 && c.max_lanes > 0, "model: max_len and max_lanes must be positive");
    const int t = c.tp_size > 0 ? c.tp_size : 1;
    LTHN_REQUIRE(c.tp_rank >= 0 && c.tp_rank < t, "model: tp_rank out of range");
    LTHN_REQUIRE(c.q_heads % t == 0 && c.kv_heads % t == 0, "model: heads must divide by the tensor-parallel degree");
    LTHN_REQUIRE((c.q_heads / t * c.head_dim) % 64 == 0 && (c.ffn / t) % 64 == 0, "model: a tensor-parallel shard must hold whole groups");
    LTHN_REQUIRE(c.vocab % t == 0, "model: vocab must divide by the tensor-parallel degree");
    return LTHN_OK;
}

static uint64_t tensor_seed(uint64_t seed, int layer, int role) {
    return seed * 1000003ull + (uint64_t)(layer + 1) * 16ull + (uint64_t)role;
}

}  // namespace lthn

// declared in codec.cu
extern "C" int32_t lthn_synth_affine_weight_shard(void* stream, uint64_t seed, float sigma, int64_t N, int64_t K,
                                                  int64_t row0, int64_t col0, int64_t Kfull, uint32_t* packed,
                                                  uint16_t* scales, uint16_t* biases);

namespace lthn {

// rows [r0, r0+n) x cols [c0, c0+k) of a host-resident packed tensor [N,K] -> device linear
static int32_t upload_shard(Model* m, Linear* dst, int64_t dst_row0, const uint8_t* packed, const uint8_t* scales,
                            const uint8_t* biases, int64_t K, int64_t r0, int64_t n, int64_t c0, int64_t k) {
    // packed: K/2 bytes per row; scales/biases: K/64*2 bytes per row
    const size_t src_pitch_p = (size_t)K / 2, src_pitch_s = (size_t)K / 64 * 2;
    const size_t dst_pitch_p = (size_t)dst->K / 2, dst_pitch_s = (size_t)dst->K / 64 * 2;
    LTHN_CUDA_TRY(cudaMemcpy2DAsync((uint8_t*)dst->wq + dst_row0 * dst_pitch_p, dst_pitch_p,
                                    packed + r0 * src_pitch_p + c0 / 2, src_pitch_p, (size_t)k / 2, (size_t)n,
                                    cudaMemcpyHostToDevice, m->stream));
    LTHN_CUDA_TRY(cudaMemcpy2DAsync((uint8_t*)dst->s + dst_row0 * dst_pitch_s, dst_pitch_s,
                                    scales + r0 * src_pitch_s + c0 / 64 * 2, src_pitch_s, (size_t)k / 64 * 2, (size_t)n,
                                    cudaMemcpyHostToDevice, m->stream));
    LTHN_CUDA_TRY(cudaMemcpy2DAsync((uint8_t*)dst->b + dst_row0 * dst_pitch_s, dst_pitch_s,
                                    biases + r0 * src_pitch_s + c0 / 64 * 2, src_pitch_s, (size_t)k / 64 * 2, (size_t)n,
                                    cudaMemcpyHostToDevice, m->stream));
    LTHN_CUDA_TRY(cudaStreamSynchronize(m->stream));  // the caller's buffers may be unmapped after return
    return LTHN_OK;
}

struct ShardPlan { Linear* dst; int64_t dst_row0, r0, n, c0, k, Nfull, Kfull; };

// Where (layer, role) lands on this rank.
static int32_t shard_plan(Model* m, int layer, int role, ShardPlan* p) {
    const auto& c = m->c;
    const int t = std::max(1, c.tp_size), r = c.tp_rank;
    const int64_t D = c.head_dim, H = c.hidden, F = c.ffn;
    Layer& L = m->layers[layer];
    switch (role) {
        case ROLE_Q: *p = {&L.qkv, 0, (int64_t)r * m->QR_l, m->QR_l, 0, H, (int64_t)c.q_heads * D, H}; break;
        case ROLE_K: *p = {&L.qkv, m->QR_l, (int64_t)r * m->KR_l, m->KR_l, 0, H, (int64_t)c.kv_heads * D, H}; break;
        case ROLE_V: *p = {&L.qkv, (int64_t)m->QR_l + m->KR_l, (int64_t)r * m->KR_l, m->KR_l, 0, H, (int64_t)c.kv_heads * D, H}; break;
        case ROLE_O: *p = {&L.o, 0, 0, H, (int64_t)r * m->QR_l, m->QR_l, H, (int64_t)c.q_heads * D}; break;
        case ROLE_GATE: *p = {&L.gate, 0, (int64_t)r * m->F_l, m->F_l, 0, H, F, H}; break;
        case ROLE_UP: *p = {&L.up, 0, (int64_t)r * m->F_l, m->F_l, 0, H, F, H}; break;
        case ROLE_DOWN: *p = {&L.down, 0, 0, H, (int64_t)r * m->F_l, m->F_l, H, F}; break;
        default: return fail(LTHN_ERR_INVALID, "model: unknown linear role");
    }
    (void)t;
    return LTHN_OK;
}

// 3..32 rows on 8-bit linears: the 8-bit form of the prefill GEMM on the bf16 rounding of the activations (the
// contract the 4-bit linears' tensor-core matvec has at these row counts); LTHN_CUDA_BATCH_F32=1 keeps the f32-grade
// general kernel
static bool batch8_on_tensor_cores(int rows) { return rows > 2 && !qmv_batch_f32(); }

// y[rows, N] = x[rows, K] W^T for one linear at its own code width (f32 in, f32 out, no fused norm or GeGLU)
static int32_t project_plain(Model* m, cudaStream_t s, const Linear& l, const float* x, float* y, int rows) {
    if (l.bits == 8 && batch8_on_tensor_cores(rows)) {
        int32_t rc = split_f32_launch(s, x, rows, l.K, 1, m->x8);
        if (rc) return rc;
        QmmCall q{m->x8, rows, l.wq, l.s, l.b, nullptr, nullptr, nullptr, l.N, l.K, y, 1};
        q.bits = 8;
        return qmm_launch(s, q);
    }
    if (l.bits == 8) return lthn_affine_qmv(s, x, LTHN_DTYPE_F32, rows, l.wq, l.s, l.b, l.N, l.K, 64, 8, y, LTHN_DTYPE_F32);
    QmvCall q{l.wq, l.s, l.b, nullptr, nullptr, nullptr, x, LTHN_DTYPE_F32, y, LTHN_DTYPE_F32, l.N, l.K, rows};
    return qmv_dispatch(s, q);
}

static int32_t all_reduce(Model* m, float* buf, size_t n) {
    if (m->c.tp_size <= 1) return LTHN_OK;
    if (!m->comm) return fail(LTHN_ERR_STATE, "model: tensor-parallel model has no communicator (call lthn_model_set_comm)");
    return nccl_check(g_nccl.AllReduce(buf, buf, n, kNcclFloat32, kNcclSum, m->comm, m->stream), "ncclAllReduce");
}

// gathers (value, index) pairs of every rank and keeps the best (ties -> lowest index)
__global__ void tp_pack_kernel(const float* v, const int32_t* idx, float* out, int rows) {
    const int r = threadIdx.x;
    if (r < rows) { out[2 * r] = v[r]; out[2 * r + 1] = __int_as_float(idx[r]); }
}
// The same gather over peer memory (no NCCL call on the decode path, so the whole step can live in
// a CUDA graph): every rank pushes its (value, index) pairs into its slot of every peer's pair
// area, signals with the exchange's sequence number, waits (bounded) for the others and picks.
// One block; protocol and counters are those of rmsnorm_gather_kernel.
__global__ void tp_pair_gather_kernel(const PairGather pg, const float* v, int32_t* idx, int rows) {
    pdl_trigger();
    pdl_wait();
    __shared__ uint32_t seq_s;
    const int tid = threadIdx.x;
    if (tid == 0) seq_s = *(volatile uint32_t*)&pg.ctr[0] + 1u;
    __syncthreads();
    const uint32_t seq = seq_s;
    for (int i = tid; i < rows * pg.t; i += blockDim.x) {
        const int r = i % rows, p = i / rows;
        float* dst = pg.pairs_out[p] + ((size_t)pg.rank * pg.max_rows + r) * 2;
        asm volatile("st.relaxed.sys.global.f32 [%0], %1;" ::"l"(dst), "f"(v[r]) : "memory");
        asm volatile("st.relaxed.sys.global.f32 [%0], %1;" ::"l"(dst + 1), "f"(__int_as_float(idx[r])) : "memory");
    }
    __threadfence_system();
    __syncthreads();
    if (tid < pg.t) {
        asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(pg.flag_out[tid] + pg.rank), "r"(seq) : "memory");
        bool ok = false;
        for (uint32_t it = 0; it < (1u << 21); ++it) {
            uint32_t f;
            asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(f) : "l"(pg.flag_in + tid) : "memory");
            if ((int32_t)(f - seq) >= 0) { ok = true; break; }
            __nanosleep(it < 64 ? 20 : 500);
        }
        if (!ok) atomicOr(pg.status, 256u);
    }
    __syncthreads();
    if (tid < rows) {
        float bv = -INFINITY; int bi = 0x7fffffff;
        for (int k = 0; k < pg.t; k++) {
            float pv, pi;
            const float* src = pg.pairs_in + ((size_t)k * pg.max_rows + tid) * 2;
            asm volatile("ld.relaxed.sys.global.f32 %0, [%1];" : "=f"(pv) : "l"(src) : "memory");
            asm volatile("ld.relaxed.sys.global.f32 %0, [%1];" : "=f"(pi) : "l"(src + 1) : "memory");
            const int i = __float_as_int(pi);
            if (pv > bv || (pv == bv && i < bi)) { bv = pv; bi = i; }
        }
        idx[tid] = bi;
    }
    __syncthreads();
    if (tid == 0) *(volatile uint32_t*)&pg.ctr[0] = seq;
}
__global__ void tp_pick_kernel(const float* gathered, int ranks, int rows, int32_t* out_idx) {
    const int r = threadIdx.x;
    if (r >= rows) return;
    float bv = -INFINITY; int bi = 0x7fffffff;
    for (int k = 0; k < ranks; k++) {
        const float v = gathered[(k * rows + r) * 2];
        const int i = __float_as_int(gathered[(k * rows + r) * 2 + 1]);
        if (v > bv || (v == bv && i < bi)) { bv = v; bi = i; }
    }
    out_idx[r] = bi;
}

// lm_head + greedy pick for rows [logit_row0, rows) of the final-normed hidden rows in xn (their
// bf16 split columns in xn_cols when `split` matches what the matvec wants): logits land in
// m->logits rows 0.., tokens in d_next[logit_row0..]. Vocab-sharded under tensor parallelism: the
// local best (value, global index) per row is gathered from all ranks.
// gemma3 layer types (model/arch/google/gemma3/gemma3.go:111-122): block i is global when (i+1) % pattern == 0
static inline int layer_window(const Model* m, int li) {
    return (m->c.sliding_window > 0 && (li + 1) % m->c.sliding_pattern != 0) ? m->c.sliding_window : 0;
}
static inline const float2* layer_rope(const Model* m, int li) { return layer_window(m, li) ? m->rope_local : m->rope; }

// An event on the model's stream that closes `phase` (-1 opens the step); a no-op unless a trace is on.
static void trace_mark(Model* m, int phase) {
    auto& t = m->trace;
    if (!t.on) return;
    if (t.used == t.ev.size()) {
        cudaEvent_t e = nullptr;
        if (cudaEventCreate(&e) != cudaSuccess) { t.on = false; return; }
        t.ev.push_back(e);
        t.ends.push_back(phase);
    }
    t.ends[t.used] = phase;
    cudaEventRecord(t.ev[t.used++], m->stream);
}
// after the step's stream synchronisation: fold the event spans into the phase totals
static void trace_collect(Model* m) {
    auto& t = m->trace;
    if (!t.on || t.used < 2) { t.used = 0; return; }
    for (size_t i = 1; i < t.used; i++) {
        float ms = 0.f;
        if (cudaEventElapsedTime(&ms, t.ev[i - 1], t.ev[i]) != cudaSuccess) continue;
        if (t.ends[i] >= 0) t.phase_us[t.ends[i]] += 1e3 * ms;
        t.gpu_us += 1e3 * ms;
    }
    t.used = 0;
    t.tokens++;
}

static int32_t lm_head_pick(Model* m, int rows, int logit_row0, int split) {
    const auto& c = m->c;
    cudaStream_t s = m->stream;
    const int H = c.hidden;
    int32_t rc;
    const int lr = rows - logit_row0;
    QmvCall hc{m->head.wq, m->head.s, m->head.b, nullptr, nullptr, nullptr, m->xn + (int64_t)logit_row0 * H, LTHN_DTYPE_F32,
               m->logits, LTHN_DTYPE_F32, m->head.N, m->head.K, lr};
    if (split > 0 && qmv_split_for(lr, LTHN_DTYPE_F32) == split) { hc.x_cols = m->xn_cols + (int64_t)logit_row0 * split * H; hc.x_split = split; }
    if ((rc = qmv_dispatch(s, hc))) return rc;
    if (c.tp_size <= 1)
        return launch_argmax(s, m->logits, lr, m->V_l, m->amax_v, m->amax_i, m->d_next + logit_row0, nullptr, 0);
    if ((rc = launch_argmax(s, m->logits, lr, m->V_l, m->amax_v, m->amax_i, m->d_next + logit_row0, m->best_v, m->v0))) return rc;
    if (m->xchg_ready) {
        LTHN_CUDA_TRY(launch_k(tp_pair_gather_kernel, dim3(1), dim3(64), 0, s, m->pairg, (const float*)m->best_v, m->d_next + logit_row0, lr));
        return LTHN_OK;
    }
    tp_pack_kernel<<<1, 32, 0, s>>>(m->best_v, m->d_next + logit_row0, m->gather, lr);
    LTHN_CUDA_TRY(cudaGetLastError());
    float* all = m->gather + 2 * kMaxRows;
    if ((rc = nccl_check(g_nccl.AllGather(m->gather, all, (size_t)2 * lr, kNcclFloat32, m->comm, s), "ncclAllGather"))) return rc;
    tp_pick_kernel<<<1, 32, 0, s>>>(all, c.tp_size, lr, m->d_next + logit_row0);
    LTHN_CUDA_TRY(cudaGetLastError());
    return LTHN_OK;
}

// One forward over `rows` (<= kMaxRows) tokens whose ids / positions / lanes are already in
// d_ids / d_pos / d_lane. max_ctx bounds pos+1 over the rows (host knowledge, sizes the
// split-KV grid). Leaves the final-normed hidden rows in xn; computes logits + greedy
// token for rows [logit_row0, rows) when want_logits.
static int32_t forward(Model* m, int rows, int max_ctx, bool want_logits, int logit_row0) {
    const auto& c = m->c;
    cudaStream_t s = m->stream;
    const int H = c.hidden, D = c.head_dim;
    int32_t rc;
    // Batch 1-2: the residual RMSNorm pairs run as the prologue of the matvec that consumes them (two
    // kernels fewer per block). The residual stream then alternates between two buffers, because
    // the CTA that stores the updated stream must not overwrite what the other CTAs of the same
    // kernel are still reading. Site 0 is the post-attention pair (consumer: gate/up), site 1 the
    // post-FFN pair (consumer: the next block's q|k|v, or the lm_head). Under tensor parallelism a
    // fused site also carries the exchange: the projection pushes its partial sums into every
    // rank's memory and the consumer waits for the peers' signals and adds the partials itself.
    const bool tp = c.tp_size > 1;
    const bool xg = m->xchg_ready;
    const bool small = rows <= 2 && (!want_logits || logit_row0 == 0);
    const bool f0 = small && (tp ? (xg && m->site_fused[0]) : m->fuse_norm);
    const bool f1 = small && (tp ? (xg && m->site_fused[1]) : m->fuse_norm);
    float* hcur = m->h;
    float* halt = m->h2;
    trace_mark(m, -1);
    if ((rc = launch_embed(s, m->d_ids, rows, m->embed.wq, m->embed.s, m->embed.b, H, c.vocab, c.embed_scale, hcur))) return rc;
    trace_mark(m, PH_EMBED);
    if (m->persist_ok && rows == 1 && (!want_logits || logit_row0 == 0)) {
        // one kernel for all blocks; it leaves the last down-projection output in a and the residual
        // stream in h2 (2*layers-1 updates alternate between h and h2), which is what the lm_head's
        // fused final norm reads
        if ((rc = launch_decode_persistent(s, m->pk, m->pk_smem))) return rc;
        trace_mark(m, PH_BLOCKS);
        if (!want_logits) return LTHN_OK;
        NormFuse nf{m->a, m->h2, m->h, m->layers[c.layers - 1].norm[NORM_POST_FF], m->final_norm, c.eps};
        QmvCall hc{m->head.wq, m->head.s, m->head.b, nullptr, nullptr, nullptr, m->xn, LTHN_DTYPE_F32, m->logits, LTHN_DTYPE_F32,
                   m->head.N, m->head.K, rows};
        hc.norm = &nf;
        if ((rc = qmv_dispatch(s, hc))) return rc;
        rc = launch_argmax(s, m->logits, rows, m->V_l, m->amax_v, m->amax_i, m->d_next, nullptr, 0);
        trace_mark(m, PH_HEAD);
        return rc;
    }
    const int split = qmv_split_for(rows, LTHN_DTYPE_F32);
    if (!f1 && (rc = launch_rmsnorm(s, hcur, nullptr, m->layers[0].norm[NORM_INPUT], nullptr, m->xn, rows, H, c.eps, 0, m->xn_cols, split))) return rc;
    int chunk_len = 0;
    const int nchunks = sdpa_chunking(max_ctx, D, &chunk_len, rows, std::max(1, m->Hkv_l));
    const size_t need = sdpa_scratch_bytes(rows, m->Hq_l, D, nchunks);
    if (nchunks > 1 && need > m->sdpa_part_bytes) return fail(LTHN_ERR_STATE, "forward: attention scratch too small");
    NormFuse nf{};
    // the fused norm of a site: partial sums from the projection (one vector, or one per rank)
    auto site_norm = [&](int site, const float* w_post, const float* w_next) {
        NormFuse n{tp ? m->x_site[site] : m->a, hcur, halt, w_post, w_next, c.eps};
        if (tp) { n.na = c.tp_size; n.a_stride = m->x_stride; n.wait = m->d_pw; }
        std::swap(hcur, halt);
        return n;
    };
    // where a row-parallel projection leaves its result
    auto site_out = [&](int site, bool fused, QmvCall& q) {
        if (!tp) return;
        if (fused) { q.npush = c.tp_size; q.push = m->d_push[site]; }
        else if (xg) q.y = m->x_part[site];
    };
    for (int li = 0; li < c.layers; li++) {
        Layer& L = m->layers[li];
        QmvCall qc{L.qkv.wq, L.qkv.s, L.qkv.b, nullptr, nullptr, nullptr, m->xn, LTHN_DTYPE_F32, m->qkv, LTHN_DTYPE_F32, L.qkv.N, L.qkv.K, rows};
        if (f1) {
            // input norm of this block, preceded (after the first block) by the previous block's post-FFN norm + residual
            if (li == 0) nf = NormFuse{nullptr, hcur, nullptr, nullptr, L.norm[NORM_INPUT], c.eps};
            else nf = site_norm(1, m->layers[li - 1].norm[NORM_POST_FF], L.norm[NORM_INPUT]);
            qc.norm = &nf;
        } else {
            qc.x_cols = m->xn_cols; qc.x_split = split;
        }
        if ((rc = qmv_dispatch(s, qc))) return rc;
        uint16_t* kc = m->kcache + (int64_t)li * m->layer_stride;
        uint16_t* vc = m->vcache + (int64_t)li * m->layer_stride;
        if (small && m->attn_fused) {
            SdpaFusedArgs fa{m->qkv, L.norm[NORM_Q], L.norm[NORM_K], layer_rope(m, li), m->d_pos, m->d_lane, kc, vc, m->lane_stride, m->att, m->sdpa_part,
                             m->att_ctr, m->Hq_l, m->Hkv_l, sdpa_item_chunks(max_ctx, D), c.max_len, c.eps, c.attn_scale};
            if ((rc = launch_sdpa_fused(s, fa, rows, D))) return rc;
        } else {
            if ((rc = launch_qknorm_rope_append(s, m->qkv, L.norm[NORM_Q], L.norm[NORM_K], layer_rope(m, li), m->d_pos, m->d_lane, m->q, kc, vc,
                                                rows, m->Hq_l, m->Hkv_l, D, c.eps, m->lane_stride, c.max_len))) return rc;
            SdpaArgs sa{m->q, kc, vc, m->d_pos, m->d_lane, m->att, m->sdpa_part, m->lane_stride, m->Hq_l, m->Hkv_l, nchunks, chunk_len, c.attn_scale};
            sa.cols = m->att_cols; sa.split = split; sa.window = layer_window(m, li);
            if ((rc = launch_sdpa_decode(s, sa, rows, D))) return rc;
        }
        QmvCall oc{L.o.wq, L.o.s, L.o.b, nullptr, nullptr, nullptr, m->att, LTHN_DTYPE_F32, m->a, LTHN_DTYPE_F32, L.o.N, L.o.K, rows};
        if (nchunks > 1 && !(small && m->attn_fused)) { oc.x_cols = m->att_cols; oc.x_split = split; }  // the merge stage wrote them
        site_out(0, f0, oc);
        if ((rc = qmv_dispatch(s, oc))) return rc;
        trace_mark(m, PH_ATTN);
        QmvCall gc{L.gate.wq, L.gate.s, L.gate.b, L.up.wq, L.up.s, L.up.b, m->xn, LTHN_DTYPE_F32, m->act, LTHN_DTYPE_F32, L.gate.N, L.gate.K, rows};
        if (f0) {
            nf = site_norm(0, L.norm[NORM_POST_ATTN], L.norm[NORM_PRE_FF]);
            gc.norm = &nf;
        } else {
            if (tp && xg) {
                if ((rc = launch_rmsnorm_gather(s, m->pg[0], hcur, L.norm[NORM_POST_ATTN], L.norm[NORM_PRE_FF], m->xn, rows, H, c.eps, m->xn_cols, split))) return rc;
            } else {
                if ((rc = all_reduce(m, m->a, (size_t)rows * H))) return rc;
                if (tp) trace_mark(m, PH_EXCHANGE);
                if ((rc = launch_rmsnorm(s, m->a, hcur, L.norm[NORM_POST_ATTN], L.norm[NORM_PRE_FF], m->xn, rows, H, c.eps, 1, m->xn_cols, split))) return rc;
            }
            gc.x_cols = m->xn_cols; gc.x_split = split;
        }
        if (L.gate.bits == 8 && L.up.bits == 8 && rows <= 2 && m->pair8_ok) {
            // both at 8 bits, one or two rows: the same fused pair (and norm prologue, when f0) on the code bytes
            gc.bits = 8;
            gc.x_cols = nullptr; gc.x_split = 0;
            if ((rc = qmv_dispatch(s, gc))) return rc;
        } else if (L.gate.bits == 8 && L.up.bits == 8 && batch8_on_tensor_cores(rows)) {
            // 3..32 rows: the pair in one pass of the 8-bit prefill GEMM
            if ((rc = split_f32_launch(s, m->xn, rows, H, 1, m->x8))) return rc;
            QmmCall g8{m->x8, rows, L.gate.wq, L.gate.s, L.gate.b, L.up.wq, L.up.s, L.up.b, L.gate.N, L.gate.K, m->act, 1};
            g8.bits = 8;
            if ((rc = qmm_launch(s, g8))) return rc;
        } else if (L.gate.bits == 8 || L.up.bits == 8) {
            // only one of the two at 8 bits (or the f32-grade batch path): separate matvecs, GeGLU in a kernel of its own
            if ((rc = project_plain(m, s, L.gate, m->xn, m->g8, rows)) || (rc = project_plain(m, s, L.up, m->xn, m->u8, rows)) ||
                (rc = launch_geglu(s, m->g8, m->u8, m->act, (int64_t)rows * L.gate.N)))
                return rc;
        } else if ((rc = qmv_dispatch(s, gc))) return rc;
        QmvCall dc{L.down.wq, L.down.s, L.down.b, nullptr, nullptr, nullptr, m->act, LTHN_DTYPE_F32, m->a, LTHN_DTYPE_F32, L.down.N, L.down.K, rows};
        site_out(1, f1, dc);
        if (L.down.bits == 8) {
            if ((rc = project_plain(m, s, L.down, m->act, m->a, rows))) return rc;
        } else if ((rc = qmv_dispatch(s, dc))) return rc;
        trace_mark(m, PH_MLP);
        const float* next_norm = li + 1 < c.layers ? m->layers[li + 1].norm[NORM_INPUT] : m->final_norm;
        if (f1) {
            // folded into the next block's QKV matvec (or the lm_head below)
        } else if (tp && xg) {
            if ((rc = launch_rmsnorm_gather(s, m->pg[1], hcur, L.norm[NORM_POST_FF], next_norm, m->xn, rows, H, c.eps, m->xn_cols, split))) return rc;
        } else {
            if ((rc = all_reduce(m, m->a, (size_t)rows * H))) return rc;
            if (tp) trace_mark(m, PH_EXCHANGE);
            if ((rc = launch_rmsnorm(s, m->a, hcur, L.norm[NORM_POST_FF], next_norm, m->xn, rows, H, c.eps, 1, m->xn_cols, split))) return rc;
        }
    }
    if (f1 && !want_logits) return LTHN_OK;
    if (f1) {
        nf = site_norm(1, m->layers[c.layers - 1].norm[NORM_POST_FF], m->final_norm);
        QmvCall hc{m->head.wq, m->head.s, m->head.b, nullptr, nullptr, nullptr, m->xn, LTHN_DTYPE_F32, m->logits, LTHN_DTYPE_F32,
                   m->head.N, m->head.K, rows};
        hc.norm = &nf;
        if ((rc = qmv_dispatch(s, hc))) return rc;
        if (!tp) {
            rc = launch_argmax(s, m->logits, rows, m->V_l, m->amax_v, m->amax_i, m->d_next, nullptr, 0);
            trace_mark(m, PH_HEAD);
            return rc;
        }
        if ((rc = launch_argmax(s, m->logits, rows, m->V_l, m->amax_v, m->amax_i, m->d_next, m->best_v, m->v0))) return rc;
        LTHN_CUDA_TRY(launch_k(tp_pair_gather_kernel, dim3(1), dim3(64), 0, s, m->pairg, (const float*)m->best_v, m->d_next, rows));
        trace_mark(m, PH_HEAD);
        return LTHN_OK;
    }
    if (!want_logits) return LTHN_OK;
    rc = lm_head_pick(m, rows, logit_row0, split);
    trace_mark(m, PH_HEAD);
    return rc;
}

static int32_t forward_full(Model* m, int rows, int max_ctx, bool want_logits, int logit_row0) {
    // kernels of a forward are chained with programmatic dependent launch: each one may start
    // (and prefetch its weights) while its predecessor drains. LTHN_CUDA_NO_PDL=1 turns it off.
    static const bool pdl = getenv("LTHN_CUDA_NO_PDL") == nullptr;
    pdl_set(pdl);
    const int32_t rc = forward(m, rows, max_ctx, want_logits, logit_row0);
    pdl_set(false);
    return rc;
}

// Prefill of one chunk on the tensor cores: `rows` (<= kPrefillRows) consecutive tokens of one
// lane starting at position pos0, ids / positions / lane in p_ids / p_pos / p_lane. The
// reference routes more than one row through affine_qmm_t (engine/metal/quant_seam_backend.go:
// 37-68) in chunks of 512 (decode/generate/generate.go:147-150); this is that path with the Metal
// engine's bf16 contract: the residual stream, norms and projection outputs stay f32, the
// activations entering a projection are rounded to bf16 (the bf16 copy the norm kernel writes,
// the attention output, the GeGLU product) and the weights are dequantised to bf16 inside
// affine_qmm. Layer order as forward(). `last` computes the logits and the greedy token of the
// chunk's final row (into row 0 of the logits buffer and d_next[0]).
static int32_t prefill_chunk(Model* m, int lane, int rows, int pos0, bool last) {
    const auto& c = m->c;
    cudaStream_t s = m->stream;
    const int H = c.hidden, D = c.head_dim;
    const bool tp = c.tp_size > 1;
    int32_t rc;
    if ((rc = launch_embed(s, m->p_ids, rows, m->embed.wq, m->embed.s, m->embed.b, H, c.vocab, c.embed_scale, m->p_h))) return rc;
    if ((rc = launch_rmsnorm(s, m->p_h, nullptr, m->layers[0].norm[NORM_INPUT], nullptr, nullptr, rows, H, c.eps, 0, m->p_xn, 1))) return rc;
    const float scale_log2e = (float)((double)c.attn_scale * 1.4426950408889634);
    for (int li = 0; li < c.layers; li++) {
        Layer& L = m->layers[li];
        QmmCall qc{m->p_xn, rows, L.qkv.wq, L.qkv.s, L.qkv.b, nullptr, nullptr, nullptr, L.qkv.N, L.qkv.K, m->p_qkv, 1};
        if ((rc = qmm_launch(s, qc))) return rc;
        uint16_t* kc = m->kcache + (int64_t)li * m->layer_stride;
        uint16_t* vc = m->vcache + (int64_t)li * m->layer_stride;
        if ((rc = launch_qknorm_rope_append(s, m->p_qkv, L.norm[NORM_Q], L.norm[NORM_K], layer_rope(m, li), m->p_pos, m->p_lane, m->p_q, kc, vc,
                                            rows, m->Hq_l, m->Hkv_l, D, c.eps, m->lane_stride, c.max_len))) return rc;
        PrefillAttnArgs pa{m->p_q, kc + (int64_t)lane * m->lane_stride, vc + (int64_t)lane * m->lane_stride, m->p_att, rows, pos0,
                           m->Hq_l, m->Hkv_l, scale_log2e};
        pa.window = layer_window(m, li);
        if ((rc = launch_prefill_attn(s, pa, D))) return rc;
        QmmCall oc{m->p_att, rows, L.o.wq, L.o.s, L.o.b, nullptr, nullptr, nullptr, L.o.N, L.o.K, m->p_a, 1};
        if ((rc = qmm_launch(s, oc))) return rc;
        if (tp && (rc = all_reduce(m, m->p_a, (size_t)rows * H))) return rc;
        if ((rc = launch_rmsnorm(s, m->p_a, m->p_h, L.norm[NORM_POST_ATTN], L.norm[NORM_PRE_FF], nullptr, rows, H, c.eps, 1, m->p_xn, 1))) return rc;
        QmmCall gc{m->p_xn, rows, L.gate.wq, L.gate.s, L.gate.b, L.up.wq, L.up.s, L.up.b, L.gate.N, L.gate.K, m->p_act, 0};
        gc.bits = L.gate.bits;  // the pair shares one width (finalize keeps other models off this path)
        if ((rc = qmm_launch(s, gc))) return rc;
        QmmCall dc{m->p_act, rows, L.down.wq, L.down.s, L.down.b, nullptr, nullptr, nullptr, L.down.N, L.down.K, m->p_a, 1};
        dc.bits = L.down.bits;
        if ((rc = qmm_launch(s, dc))) return rc;
        if (tp && (rc = all_reduce(m, m->p_a, (size_t)rows * H))) return rc;
        const bool final_layer = li + 1 == c.layers;
        const float* next_norm = final_layer ? m->final_norm : m->layers[li + 1].norm[NORM_INPUT];
        if ((rc = launch_rmsnorm(s, m->p_a, m->p_h, L.norm[NORM_POST_FF], next_norm, final_layer && last ? m->p_xnf : nullptr, rows, H,
                                 c.eps, 1, final_layer ? nullptr : m->p_xn, final_layer ? 0 : 1))) return rc;
    }
    if (!last) return LTHN_OK;
    LTHN_CUDA_TRY(cudaMemcpyAsync(m->xn, m->p_xnf + (int64_t)(rows - 1) * H, (size_t)H * sizeof(float), cudaMemcpyDeviceToDevice, s));
    return lm_head_pick(m, 1, 0, 0);
}

// One decode step for `rows` lanes (ids / positions / lanes already in the device buffers),
// every row producing a token. The first call per row count runs eagerly (first use of a
// kernel may allocate scratch), the second captures the step into a CUDA graph, later calls
// replay it: ~210 launches per token become one graph launch. The split-KV grid is sized for
// max_len so the graph does not depend on the current context length. LTHN_CUDA_NO_GRAPH=1
// keeps the eager path.
static int32_t decode_step(Model* m, int rows) {
    if (m->trace.on) return forward_full(m, rows, m->c.max_len, true, 0);  // events between the phases need separate launches
    if (m->step_graph[rows]) {
        LTHN_CUDA_TRY(cudaGraphLaunch(m->step_graph[rows], m->stream));
        return LTHN_OK;
    }
    if (m->graphs_off || !m->step_warm[rows]) {
        m->step_warm[rows] = true;
        return forward_full(m, rows, m->c.max_len, true, 0);
    }
    LTHN_CUDA_TRY(cudaStreamBeginCapture(m->stream, cudaStreamCaptureModeThreadLocal));
    const int32_t rc = forward_full(m, rows, m->c.max_len, true, 0);
    cudaGraph_t g = nullptr;
    const cudaError_t e = cudaStreamEndCapture(m->stream, &g);
    cudaGraphExec_t ex = nullptr;
    if (rc == LTHN_OK && e == cudaSuccess && g && cudaGraphInstantiate(&ex, g, 0) == cudaSuccess) {
        cudaGraphDestroy(g);
        m->step_graph[rows] = ex;
        LTHN_CUDA_TRY(cudaGraphLaunch(ex, m->stream));
        return LTHN_OK;
    }
    if (g) cudaGraphDestroy(g);
    cudaGetLastError();
    clear_error();
    m->graphs_off = true;  // capture is not possible here: stay eager
    return forward_full(m, rows, m->c.max_len, true, 0);
}

// ---- lanes / sessions ------------------------------------------------------------------
struct Lane {
    int id = -1;       // KV lane index in the model
    int pos = 0;       // tokens in the cache
    int pending = -1;  // generated token not yet fed
    bool have_next = false;  // d_next of the last forward holds this lane's next token
    int next_tok = -1;
    uint64_t logits_serial = 0;  // Model::logits_serial of the forward that produced this lane's logits
    int logits_row = 0;          // its row in the logits buffer
    // lane-set bookkeeping
    int handle = 0, produced = 0, max_new = 0;
    bool terminal = false;
    std::vector<int32_t> stop;
    std::shared_ptr<struct SampleState> samp;  // set for lanes that sample (LaneSpec.Sampler)
};

// Per-lane (or per-call) sampling state: the reference keeps one Sampler per request and a history
// of the tokens generated so far for the repeat penalty (model/token.go:263-305).
struct SampleState {
    HostSampler own;            // lane sets: the lane's own RNG stream
    HostSampler* rng = nullptr; // the stream in use (sessions: the caller's sampler)
    lthn_sample_params p{};
    std::vector<int32_t> suppress, history;
    int generated = 0;
};
constexpr int kSampleListCap = 1 << 16;

static int32_t sample_workspace(Model* m) {
    if (m->s_bits) return LTHN_OK;
    int32_t rc;
    const size_t t = (size_t)std::max(1, m->c.tp_size);
    if ((rc = dalloc(m, &m->s_bits, (size_t)m->V_l)) || (rc = dalloc(m, &m->s_cbits, (size_t)SAMPLE_KMAX)) ||
        (rc = dalloc(m, &m->s_cidx, (size_t)SAMPLE_KMAX)) || (rc = dalloc(m, &m->s_lists, (size_t)2 * kSampleListCap)) ||
        (rc = dalloc(m, &m->s_gather, 2 * (size_t)SAMPLE_KMAX * (1 + t))))
        return rc;
    return LTHN_OK;
}

__global__ void sample_pack_kernel(const int32_t* idx, const uint16_t* bits, int k, float* out) {
    const int i = threadIdx.x;
    if (i < k) { out[2 * i] = __uint_as_float((uint32_t)bits[i] << 16); out[2 * i + 1] = __int_as_float(idx[i]); }
}

// One token for the row `row` of the model's logits buffer (which must still hold that lane's
// logits). stop: the request's stop tokens (suppressed until min_tokens_before_stop tokens exist).
static int32_t sample_row(Model* m, int row, SampleState& st, const std::vector<int32_t>& stop, int32_t* token) {
    int32_t rc;
    if ((rc = sample_workspace(m))) return rc;
    cudaStream_t s = m->stream;
    const auto& c = m->c;
    lthn_sample_params p = st.p;
    std::vector<int32_t> sup = st.suppress;
    if (p.min_tokens_before_stop > 0 && st.generated < p.min_tokens_before_stop)  // appendSuppressionTokens (model/token.go:645-655)
        for (int32_t tk : stop) if (std::find(sup.begin(), sup.end(), tk) == sup.end()) sup.push_back(tk);
    p.suppress = sup.data();
    p.n_suppress = (int)sup.size();
    const bool penal = p.repeat_penalty > 1.0f && !st.history.empty();
    const int nh = penal ? (int)st.history.size() : 0;
    if (nh > kSampleListCap || (int)sup.size() > kSampleListCap) return fail(LTHN_ERR_INVALID, "sampler: history or suppress list longer than 65536 ids");
    if (nh) LTHN_CUDA_TRY(cudaMemcpyAsync(m->s_lists, st.history.data(), (size_t)nh * 4, cudaMemcpyHostToDevice, s));
    if (!sup.empty()) LTHN_CUDA_TRY(cudaMemcpyAsync(m->s_lists + kSampleListCap, sup.data(), sup.size() * 4, cudaMemcpyHostToDevice, s));
    const float* logits = m->logits + (size_t)row * m->V_l;
    if ((rc = sample_prepare_device(s, logits, m->V_l, m->v0, m->s_lists, nh, p.repeat_penalty, m->s_lists + kSampleListCap, (int)sup.size(), m->s_bits))) return rc;
    // the lists were applied on the device: the host sampler sees plain logits
    lthn_sample_params hp = p;
    hp.suppress = nullptr; hp.n_suppress = 0; hp.repeat_penalty = 0;
    const bool greedy = p.temperature <= 0 && p.min_p <= 0;
    const int k = greedy ? 1 : p.top_k;
    if (k >= 1 && k <= SAMPLE_KMAX && k < c.vocab) {
        const int kl = std::min(k, m->V_l);
        if ((rc = sample_topk_device(s, m->s_bits, 1, m->V_l, kl, m->v0, m->s_cidx, m->s_cbits))) return rc;
        std::vector<std::pair<uint16_t, int32_t>> cand;
        if (c.tp_size > 1) {
            // every rank contributes its shard's best kl; all ranks merge the same list and draw the same token
            sample_pack_kernel<<<1, SAMPLE_KMAX, 0, s>>>(m->s_cidx, m->s_cbits, kl, m->s_gather);
            LTHN_CUDA_TRY(cudaGetLastError());
            float* all = m->s_gather + 2 * SAMPLE_KMAX;
            if ((rc = nccl_check(g_nccl.AllGather(m->s_gather, all, (size_t)2 * kl, kNcclFloat32, m->comm, s), "ncclAllGather"))) return rc;
            std::vector<float> h((size_t)2 * kl * c.tp_size);
            LTHN_CUDA_TRY(cudaMemcpyAsync(h.data(), all, h.size() * 4, cudaMemcpyDeviceToHost, s));
            LTHN_CUDA_TRY(cudaStreamSynchronize(s));
            for (size_t i = 0; i < h.size() / 2; i++) {
                uint32_t vb, ib;
                memcpy(&vb, &h[2 * i], 4); memcpy(&ib, &h[2 * i + 1], 4);
                cand.emplace_back((uint16_t)(vb >> 16), (int32_t)ib);
            }
        } else {
            std::vector<int32_t> hi(kl);
            std::vector<uint16_t> hb(kl);
            LTHN_CUDA_TRY(cudaMemcpyAsync(hi.data(), m->s_cidx, (size_t)kl * 4, cudaMemcpyDeviceToHost, s));
            LTHN_CUDA_TRY(cudaMemcpyAsync(hb.data(), m->s_cbits, (size_t)kl * 2, cudaMemcpyDeviceToHost, s));
            LTHN_CUDA_TRY(cudaStreamSynchronize(s));
            for (int i = 0; i < kl; i++) cand.emplace_back(hb[i], hi[i]);
        }
        // best first: value descending, id ascending (the order a stable descending sort of the row gives)
        std::sort(cand.begin(), cand.end(), [](const std::pair<uint16_t, int32_t>& a, const std::pair<uint16_t, int32_t>& b) {
            const float va = bf16_bits_to_f32(a.first), vb = bf16_bits_to_f32(b.first);
            if (va != vb) return va > vb;
            return a.second < b.second;
        });
        if ((int)cand.size() > k) cand.resize(k);
        std::vector<uint16_t> cb(cand.size());
        std::vector<int32_t> ci(cand.size());
        for (size_t i = 0; i < cand.size(); i++) { cb[i] = cand[i].first; ci[i] = cand[i].second; }
        return st.rng->sample(cb.data(), ci.data(), (int)cand.size(), hp, token);
    }
    if (c.tp_size > 1) return fail(LTHN_ERR_INVALID, "sampler: a tensor-parallel model samples through the device top-k window: set 1 <= top_k <= 256");
    m->s_host_bits.resize((size_t)m->V_l);
    LTHN_CUDA_TRY(cudaMemcpyAsync(m->s_host_bits.data(), m->s_bits, (size_t)m->V_l * 2, cudaMemcpyDeviceToHost, s));
    LTHN_CUDA_TRY(cudaStreamSynchronize(s));
    return st.rng->sample(m->s_host_bits.data(), nullptr, m->V_l, hp, token);
}

static int lane_acquire(Model* m) {
    std::lock_guard<std::mutex> lk(m->mu);
    for (size_t i = 0; i < m->lane_used.size(); i++)
        if (!m->lane_used[i]) { m->lane_used[i] = 1; return (int)i; }
    return -1;
}
static void lane_release(Model* m, int id) {
    std::lock_guard<std::mutex> lk(m->mu);
    if (id >= 0 && id < (int)m->lane_used.size()) m->lane_used[id] = 0;
}

// Feeds `n` tokens of one lane (prefill / append), kMaxRows at a time. The greedy token
// after the last one lands in lane->next_tok.
static int32_t feed_lane(Model* m, Lane* ln, const int32_t* ids, int n) {
    LTHN_REQUIRE(n > 0, "session: no tokens to feed");
    LTHN_REQUIRE(ln->pos + n <= m->c.max_len, "session: context length exceeded");
    for (int i = 0; i < n; i++) LTHN_REQUIRE(ids[i] >= 0 && ids[i] < m->c.vocab, "session: token id outside the vocabulary");
    std::lock_guard<std::mutex> lk(m->mu);
    int32_t rc;
    if (m->prefill_tc && n > kMaxRows) {
        // more rows than one decode forward takes: chunks of kPrefillRows through affine_qmm and the causal prefill attention
        for (int off = 0; off < n; off += m->prefill_rows) {
            const int rows = std::min(m->prefill_rows, n - off);
            int32_t* hp = m->p_pinned;
            for (int r = 0; r < rows; r++) { hp[r] = ids[off + r]; hp[kPrefillRows + r] = ln->pos + r; hp[2 * kPrefillRows + r] = ln->id; }
            LTHN_CUDA_TRY(cudaMemcpyAsync(m->p_ids, hp, 3 * kPrefillRows * 4, cudaMemcpyHostToDevice, m->stream));
            const bool last = off + rows >= n;
            if ((rc = prefill_chunk(m, ln->id, rows, ln->pos, last))) return rc;
            ln->pos += rows;
            if (last) {
                LTHN_CUDA_TRY(cudaMemcpyAsync(m->h_pinned + 3 * kMaxRows, m->d_next, 4, cudaMemcpyDeviceToHost, m->stream));
                if ((rc = device_status_read_async(m->stream, (uint32_t*)(m->h_pinned + 4 * kMaxRows)))) return rc;
            }
            LTHN_CUDA_TRY(cudaStreamSynchronize(m->stream));  // the pinned staging is reused by the next chunk
        }
        ln->next_tok = m->h_pinned[3 * kMaxRows];
        ln->have_next = true;
        ln->pending = -1;
        ln->logits_serial = ++m->logits_serial;
        ln->logits_row = 0;
        return device_status_judge((uint32_t)m->h_pinned[4 * kMaxRows], m->stream);
    }
    for (int off = 0; off < n; off += kMaxRows) {
        const int rows = std::min(kMaxRows, n - off);
        int32_t* hp = m->h_pinned;
        for (int r = 0; r < rows; r++) { hp[r] = ids[off + r]; hp[kMaxRows + r] = ln->pos + r; hp[2 * kMaxRows + r] = ln->id; }
        LTHN_CUDA_TRY(cudaMemcpyAsync(m->d_ids, hp, 3 * kMaxRows * 4, cudaMemcpyHostToDevice, m->stream));
        const bool last = off + rows >= n;
        if (n == 1) rc = decode_step(m, 1);
        else rc = forward_full(m, rows, ln->pos + rows, last, rows - 1);
        if (rc) return rc;
        ln->pos += rows;
        if (last) {
            LTHN_CUDA_TRY(cudaMemcpyAsync(hp + 3 * kMaxRows, m->d_next + rows - 1, 4, cudaMemcpyDeviceToHost, m->stream));
            if ((rc = device_status_read_async(m->stream, (uint32_t*)(hp + 4 * kMaxRows)))) return rc;
        }
        LTHN_CUDA_TRY(cudaStreamSynchronize(m->stream));  // the pinned staging is reused by the next chunk
        if (n == 1) trace_collect(m); else m->trace.used = 0;  // the tracer follows decode steps, not prompts
    }
    ln->next_tok = m->h_pinned[3 * kMaxRows];
    ln->have_next = true;
    ln->pending = -1;
    ln->logits_serial = ++m->logits_serial;
    ln->logits_row = 0;
    return device_status_judge((uint32_t)m->h_pinned[4 * kMaxRows], m->stream);
}

struct Session { Model* m; Lane lane; };
struct LaneSet {
    Model* m;
    int max_lanes;
    std::vector<Lane> lanes;
    int next_handle = 1;
    uint64_t forwards = 0;
};

}  // namespace lthn

using namespace lthn;

extern "C" {

// ---- tensor-parallel communicator ---------------------------------------------------------
int32_t lthn_tp_unique_id(void* out128) {
    clear_error();
    LTHN_REQUIRE(out128 != nullptr, "lthn_tp_unique_id: out is NULL");
    int32_t rc = nccl_load();
    if (rc) return rc;
    return nccl_check(g_nccl.GetUniqueId(out128), "ncclGetUniqueId");
}
int32_t lthn_tp_init(int32_t rank, int32_t world, const void* id128, void** comm) {
    clear_error();
    LTHN_REQUIRE(comm && id128 && world > 0 && rank >= 0 && rank < world, "lthn_tp_init: bad arguments");
    int32_t rc = nccl_load();
    if (rc) return rc;
    UniqueId id;
    memcpy(&id, id128, sizeof(id));
    return nccl_check(g_nccl.CommInitRank(comm, world, id, rank), "ncclCommInitRank");
}
int32_t lthn_tp_destroy(void* comm) {
    clear_error();
    if (!comm) return LTHN_OK;
    return nccl_check(g_nccl.CommDestroy(comm), "ncclCommDestroy");
}

// ---- model ----------------------------------------------------------------------------------
int32_t lthn_model_create(const lthn_model_config* cfg, void** model) {
    clear_error();
    LTHN_REQUIRE(cfg && model, "lthn_model_create: NULL argument");
    lthn_model_config c = *cfg;
    if (c.tp_size <= 0) c.tp_size = 1;
    if (c.eps <= 0) c.eps = 1e-6f;
    if (c.rope_base <= 0) c.rope_base = 10000.0f;
    if (c.sliding_window < 0) c.sliding_window = 0;
    if (c.sliding_pattern <= 0) c.sliding_pattern = 6;   // gemma3: every sixth block is global
    if (c.rope_local_base <= 0) c.rope_local_base = 10000.0f;
    if (c.attn_scale <= 0) c.attn_scale = (float)(1.0 / std::sqrt((double)c.head_dim));  // gemma3.go:150
    if (c.embed_scale <= 0)  // bf16(sqrt(hidden)), hip_gemma4_q4_layer.go:2757-2763
        c.embed_scale = bf16_bits_to_f32(f32_to_bf16_bits((float)std::sqrt((double)c.hidden)));
    int32_t rc = model_validate(c);
    if (rc) return rc;
    Model* m = new Model();
    m->c = c;
    m->graphs_off = getenv("LTHN_CUDA_NO_GRAPH") != nullptr;
    const int t = c.tp_size;
    m->Hq_l = c.q_heads / t; m->Hkv_l = c.kv_heads / t;
    m->QR_l = m->Hq_l * c.head_dim; m->KR_l = m->Hkv_l * c.head_dim;
    m->F_l = c.ffn / t; m->V_l = c.vocab / t; m->v0 = c.tp_rank * m->V_l;
    m->layers.resize(c.layers);
    cudaError_t e = cudaStreamCreateWithFlags(&m->stream, cudaStreamNonBlocking);
    if (e != cudaSuccess) { delete m; return cuda_fail(e, "cudaStreamCreate"); }
    auto bail = [&](int32_t code) {
        const std::string keep = lthn_last_error();
        for (void* p : m->allocs) cudaFree(p);
        if (m->h_pinned) cudaFreeHost(m->h_pinned);
        if (m->p_pinned) cudaFreeHost(m->p_pinned);
        cudaStreamDestroy(m->stream);
        delete m;
        return fail(code, keep);
    };
    const int64_t H = c.hidden;
    for (auto& L : m->layers) {
        if ((rc = linear_alloc(m, &L.qkv, (int64_t)m->QR_l + 2 * m->KR_l, H))) return bail(rc);
        if ((rc = linear_alloc(m, &L.o, H, m->QR_l))) return bail(rc);
        if ((rc = linear_alloc(m, &L.gate, m->F_l, H))) return bail(rc);
        if ((rc = linear_alloc(m, &L.up, m->F_l, H))) return bail(rc);
        if ((rc = linear_alloc(m, &L.down, H, m->F_l))) return bail(rc);
        for (int i = 0; i < NORM_COUNT; i++)
            if ((rc = dalloc(m, &L.norm[i], (size_t)(i >= NORM_Q ? c.head_dim : H)))) return bail(rc);
    }
    if ((rc = linear_alloc(m, &m->embed, c.vocab, H))) return bail(rc);
    m->head = m->embed;
    m->head.N = m->V_l;
    m->head.wq = m->embed.wq + (int64_t)m->v0 * (H / 8);
    m->head.s = m->embed.s + (int64_t)m->v0 * (H / 64);
    m->head.b = m->embed.b + (int64_t)m->v0 * (H / 64);
    if ((rc = dalloc(m, &m->final_norm, (size_t)H))) return bail(rc);
    // RoPE tables, f64 on the host exactly as hipReferenceRoPENeoXWithFrequencyDimScale: one for the global
    // blocks and, with a sliding window, one with the local base for the sliding blocks
    for (int local = 0; local < (c.sliding_window > 0 ? 2 : 1); local++) {
        const int half = c.head_dim / 2;
        const double base = local ? (double)c.rope_local_base : (double)c.rope_base;
        std::vector<float2> tab((size_t)c.max_len * half);
        for (int p = 0; p < c.max_len; p++)
            for (int i = 0; i < half; i++) {
                const double freq = 1.0 / std::pow(base, (double)(2 * i) / (double)c.head_dim);
                const double angle = (double)p * freq * 1.0;
                tab[(size_t)p * half + i] = make_float2((float)std::cos(angle), (float)std::sin(angle));
            }
        float2** dst = local ? &m->rope_local : &m->rope;
        if ((rc = dalloc(m, dst, tab.size()))) return bail(rc);
        e = cudaMemcpy(*dst, tab.data(), tab.size() * sizeof(float2), cudaMemcpyHostToDevice);
        if (e != cudaSuccess) { cuda_fail(e, "rope table upload"); return bail(LTHN_ERR_CUDA); }
    }
    m->layer_stride = (int64_t)c.max_len * m->KR_l;
    m->lane_stride = (int64_t)c.layers * m->layer_stride;
    const size_t kv_elems = (size_t)c.max_lanes * m->lane_stride;
    if ((rc = dalloc(m, &m->kcache, kv_elems))) return bail(rc);
    if ((rc = dalloc(m, &m->vcache, kv_elems))) return bail(rc);
    m->lane_used.assign(c.max_lanes, 0);
    const size_t R = kMaxRows;
    // ids / positions / lanes of a forward sit in one block, so one copy stages them
    if ((rc = dalloc(m, &m->d_ids, 3 * R)) ||
        (rc = dalloc(m, &m->d_next, R)) || (rc = dalloc(m, &m->h, R * H)) || (rc = dalloc(m, &m->h2, R * H)) || (rc = dalloc(m, &m->xn, R * H)) ||
        (rc = dalloc(m, &m->qkv, R * (m->QR_l + 2 * m->KR_l))) || (rc = dalloc(m, &m->q, R * m->QR_l)) ||
        (rc = dalloc(m, &m->att, R * m->QR_l)) || (rc = dalloc(m, &m->a, R * H)) || (rc = dalloc(m, &m->act, R * m->F_l)) ||
        (rc = dalloc(m, &m->xn_cols, R * 3 * H)) || (rc = dalloc(m, &m->att_cols, R * 3 * m->QR_l)) ||
        (rc = dalloc(m, &m->logits, R * m->V_l)) || (rc = dalloc(m, &m->amax_v, R * ARGMAX_BLOCKS)) ||
        (rc = dalloc(m, &m->amax_i, R * ARGMAX_BLOCKS)) || (rc = dalloc(m, &m->best_v, R)) ||
        (rc = dalloc(m, &m->gather, 2 * R * (1 + (size_t)c.tp_size))))
        return bail(rc);
    m->d_pos = m->d_ids + R;
    m->d_lane = m->d_ids + 2 * R;
    {
        const int nch = sdpa_item_chunks(c.max_len, c.head_dim);  // the finest chunking any attention path uses
        m->sdpa_part_bytes = sdpa_scratch_bytes(kMaxRows, m->Hq_l, c.head_dim, nch);
        if ((rc = dalloc(m, &m->sdpa_part, m->sdpa_part_bytes / sizeof(float) + 64))) return bail(rc);
    }
    e = cudaHostAlloc((void**)&m->h_pinned, 4 * kMaxRows * sizeof(int32_t) + 256, cudaHostAllocDefault);
    if (e != cudaSuccess) { cuda_fail(e, "cudaHostAlloc"); return bail(LTHN_ERR_CUDA); }
    {
        // LTHN_CUDA_PREFILL_F32=1 keeps every prompt on the f32 decode kernels (32 rows per forward);
        // the tensor-core prefill attention serves head_dim up to 256
        const char* env = getenv("LTHN_CUDA_PREFILL_F32");
        m->prefill_tc = !(env && env[0] == '1') && c.head_dim <= 256 && c.max_len > kMaxRows;
        // LTHN_CUDA_PREFILL_CHUNK=n: smaller chunks (64..2048 rows), e.g. to bound the workspace
        const char* ch = getenv("LTHN_CUDA_PREFILL_CHUNK");
        const int want = ch ? atoi(ch) : kPrefillRows;
        m->prefill_rows = std::max(64, std::min(kPrefillRows, want));
    }
    if (m->prefill_tc) {
        const size_t P = (size_t)std::min(m->prefill_rows, c.max_len);
        const size_t QKV = (size_t)m->QR_l + 2 * m->KR_l;
        if ((rc = dalloc(m, &m->p_ids, 3 * (size_t)kPrefillRows)) || (rc = dalloc(m, &m->p_h, P * H)) ||
            (rc = dalloc(m, &m->p_xn, P * H)) || (rc = dalloc(m, &m->p_xnf, P * H)) || (rc = dalloc(m, &m->p_qkv, P * QKV)) ||
            (rc = dalloc(m, &m->p_q, P * m->QR_l)) || (rc = dalloc(m, &m->p_att, P * m->QR_l)) ||
            (rc = dalloc(m, &m->p_a, P * H)) || (rc = dalloc(m, &m->p_act, P * m->F_l)))
            return bail(rc);
        m->p_pos = m->p_ids + kPrefillRows;
        m->p_lane = m->p_ids + 2 * kPrefillRows;
        e = cudaHostAlloc((void**)&m->p_pinned, 3 * kPrefillRows * sizeof(int32_t), cudaHostAllocDefault);
        if (e != cudaSuccess) { cuda_fail(e, "cudaHostAlloc"); return bail(LTHN_ERR_CUDA); }
    }
    *model = m;
    return LTHN_OK;
}

int32_t lthn_model_set_comm(void* model, void* comm) {
    clear_error();
    LTHN_REQUIRE(model != nullptr, "lthn_model_set_comm: model is NULL");
    ((Model*)model)->comm = comm;
    return LTHN_OK;
}

int32_t lthn_model_upload_linear(void* model, int32_t layer, int32_t role, const void* packed, const void* scales,
                                 const void* biases, int64_t N, int64_t K) {
    clear_error();
    Model* m = (Model*)model;
    LTHN_REQUIRE(m && packed && scales && biases, "lthn_model_upload_linear: NULL argument");
    if (layer < 0) {  // token embedding / tied lm_head, replicated
        LTHN_REQUIRE(N == m->c.vocab && K == m->c.hidden, "lthn_model_upload_linear: embedding must be [vocab, hidden]");
        int32_t rc = upload_shard(m, &m->embed, 0, (const uint8_t*)packed, (const uint8_t*)scales, (const uint8_t*)biases, K, 0, N, 0, K);
        if (rc == LTHN_OK) m->have_embed = true;
        return rc;
    }
    LTHN_REQUIRE(layer < m->c.layers, "lthn_model_upload_linear: layer out of range");
    ShardPlan p;
    int32_t rc = shard_plan(m, layer, role, &p);
    if (rc) return rc;
    LTHN_REQUIRE(N == p.Nfull && K == p.Kfull, "lthn_model_upload_linear: tensor shape does not match the model configuration");
    LTHN_REQUIRE(p.dst->bits == 4, "lthn_model_upload_linear: this linear was uploaded with 8-bit codes");
    rc = upload_shard(m, p.dst, p.dst_row0, (const uint8_t*)packed, (const uint8_t*)scales, (const uint8_t*)biases, K, p.r0, p.n, p.c0, p.k);
    if (rc == LTHN_OK) m->layers[layer].have[role] = true;
    return rc;
}

// A linear at its own code width. 4 bits: lthn_model_upload_linear. 8 bits (group 64): the MLP projections of a
// mixed-precision pack on one GPU; the linear's buffers are replaced by ones of the wider pitch.
int32_t lthn_model_upload_linear_bits(void* model, int32_t layer, int32_t role, const void* packed, const void* scales,
                                      const void* biases, int64_t N, int64_t K, int32_t bits) {
    if (bits == 4) return lthn_model_upload_linear(model, layer, role, packed, scales, biases, N, K);
    clear_error();
    Model* m = (Model*)model;
    LTHN_REQUIRE(m && packed && scales && biases, "lthn_model_upload_linear_bits: NULL argument");
    LTHN_REQUIRE(bits == 8, "lthn_model_upload_linear_bits: a linear holds 4-bit or 8-bit codes");
    LTHN_REQUIRE(!m->finalized, "lthn_model_upload_linear_bits: the model is finalized");
    LTHN_REQUIRE(m->c.tp_size <= 1, "lthn_model_upload_linear_bits: 8-bit linears are served on one GPU only");
    LTHN_REQUIRE(layer >= 0 && layer < m->c.layers, "lthn_model_upload_linear_bits: layer out of range");
    LTHN_REQUIRE(role == ROLE_GATE || role == ROLE_UP || role == ROLE_DOWN,
                 "lthn_model_upload_linear_bits: only the MLP projections (gate, up, down) take 8-bit codes");
    ShardPlan p;
    int32_t rc = shard_plan(m, layer, role, &p);
    if (rc) return rc;
    LTHN_REQUIRE(N == p.Nfull && K == p.Kfull, "lthn_model_upload_linear_bits: tensor shape does not match the model configuration");
    Linear* l = p.dst;
    if (l->bits != 8) {
        // swap the 4-bit buffers for 8-bit ones
        for (void* old : {(void*)l->wq, (void*)l->s, (void*)l->b}) {
            auto it = std::find(m->allocs.begin(), m->allocs.end(), old);
            if (it != m->allocs.end()) m->allocs.erase(it);
            LTHN_CUDA_TRY(cudaFree(old));
        }
        l->wq = nullptr; l->s = nullptr; l->b = nullptr;
        m->weight_bytes -= (uint64_t)N * K * 9 / 16;
        if ((rc = dalloc(m, &l->wq, (size_t)N * K / 4)) || (rc = dalloc(m, &l->s, (size_t)N * K / 64)) ||
            (rc = dalloc(m, &l->b, (size_t)N * K / 64)))
            return rc;
        m->weight_bytes += (uint64_t)N * K * 17 / 16;
        l->bits = 8;
    }
    if (!m->g8) {
        if ((rc = dalloc(m, &m->g8, (size_t)kMaxRows * m->F_l)) || (rc = dalloc(m, &m->u8, (size_t)kMaxRows * m->F_l)) ||
            (rc = dalloc(m, &m->x8, (size_t)kMaxRows * std::max<int64_t>(m->c.hidden, m->F_l))))
            return rc;
    }
    m->mixed = true;
    const size_t sg = (size_t)N * K / 64 * 2;
    LTHN_CUDA_TRY(cudaMemcpyAsync(l->wq, packed, (size_t)N * K, cudaMemcpyHostToDevice, m->stream));
    LTHN_CUDA_TRY(cudaMemcpyAsync(l->s, scales, sg, cudaMemcpyHostToDevice, m->stream));
    LTHN_CUDA_TRY(cudaMemcpyAsync(l->b, biases, sg, cudaMemcpyHostToDevice, m->stream));
    LTHN_CUDA_TRY(cudaStreamSynchronize(m->stream));  // the caller's buffers may be unmapped after return
    m->layers[layer].have[role] = true;
    return LTHN_OK;
}

int32_t lthn_model_upload_norm(void* model, int32_t layer, int32_t role, const float* w, int64_t n) {
    clear_error();
    Model* m = (Model*)model;
    LTHN_REQUIRE(m && w, "lthn_model_upload_norm: NULL argument");
    float* dst;
    int64_t want;
    if (layer < 0) { dst = m->final_norm; want = m->c.hidden; }
    else {
        LTHN_REQUIRE(layer < m->c.layers && role >= 0 && role < NORM_COUNT, "lthn_model_upload_norm: layer/role out of range");
        dst = m->layers[layer].norm[role];
        want = role >= NORM_Q ? m->c.head_dim : m->c.hidden;
    }
    LTHN_REQUIRE(n == want, "lthn_model_upload_norm: wrong length");
    LTHN_CUDA_TRY(cudaMemcpy(dst, w, (size_t)n * 4, cudaMemcpyHostToDevice));
    return LTHN_OK;
}

// Fills every tensor with the seeded synthetic source: linear (layer, role) is the
// [N,K] tensor of stream seed*1000003 + (layer+1)*16 + role (embedding: layer = -1,
// role 0) quantised with the reference rule; norm weights are 1 (zero stored weight
// under the gemma (1+w) fold, model/norm_bias.go).
int32_t lthn_model_synthesize(void* model, uint64_t seed, float sigma) {
    clear_error();
    Model* m = (Model*)model;
    LTHN_REQUIRE(m != nullptr, "lthn_model_synthesize: model is NULL");
    LTHN_REQUIRE(!m->mixed, "lthn_model_synthesize: the synthetic tensors are 4-bit; call it before uploading 8-bit linears");
    int32_t rc;
    const auto& c = m->c;
    for (int li = 0; li < c.layers; li++) {
        for (int role = 0; role < ROLE_COUNT; role++) {
            ShardPlan p;
            if ((rc = shard_plan(m, li, role, &p))) return rc;
            Linear* d = p.dst;
            rc = lthn_synth_affine_weight_shard(m->stream, tensor_seed(seed, li, role), sigma, p.n, p.k, p.r0, p.c0, p.Kfull,
                                                d->wq + p.dst_row0 * (d->K / 8), d->s + p.dst_row0 * (d->K / 64),
                                                d->b + p.dst_row0 * (d->K / 64));
            if (rc) return rc;
            m->layers[li].have[role] = true;
        }
    }
    if ((rc = lthn_synth_affine_weight_shard(m->stream, tensor_seed(seed, -1, 0), sigma, c.vocab, c.hidden, 0, 0, c.hidden,
                                             m->embed.wq, m->embed.s, m->embed.b))) return rc;
    m->have_embed = true;
    std::vector<float> ones((size_t)std::max(c.hidden, c.head_dim), 1.0f);
    for (int li = 0; li < c.layers; li++)
        for (int i = 0; i < NORM_COUNT; i++)
            LTHN_CUDA_TRY(cudaMemcpyAsync(m->layers[li].norm[i], ones.data(), (size_t)(i >= NORM_Q ? c.head_dim : c.hidden) * 4,
                                          cudaMemcpyHostToDevice, m->stream));
    LTHN_CUDA_TRY(cudaMemcpyAsync(m->final_norm, ones.data(), (size_t)c.hidden * 4, cudaMemcpyHostToDevice, m->stream));
    LTHN_CUDA_TRY(cudaStreamSynchronize(m->stream));
    return LTHN_OK;
}

// Maps every rank's exchange buffer into every other rank (CUDA IPC; one process per GPU) so that
// the residual RMSNorm can add the ranks' partial sums straight from peer memory. Handles travel
// through an NCCL all-gather. Any rank that cannot map a peer makes all ranks keep the NCCL
// all-reduce path (agreed with an all-reduce of a success flag). LTHN_CUDA_TP_NCCL=1 forces that path.
static int32_t xchg_setup(Model* m) {
    const auto& c = m->c;
    const int t = c.tp_size;
    if (t < 2 || t > 8 || c.hidden > 8192) return LTHN_OK;
    const char* env = getenv("LTHN_CUDA_TP_NCCL");
    const bool want = !(env && env[0] == '1');
    const size_t flag_bytes = 256;
    const size_t part_bytes = ((size_t)kMaxRows * c.hidden * sizeof(float) + 255) / 256 * 256;
    const size_t pair_bytes = ((size_t)8 * kMaxRows * 2 * sizeof(float) + 255) / 256 * 256;
    const size_t site_bytes = 8 * part_bytes;  // one slot per rank
    const size_t total = flag_bytes + 2 * site_bytes + pair_bytes;
    float ok = want ? 1.f : 0.f;
    cudaIpcMemHandle_t mine{};
    if (ok > 0.f) {
        if (cudaMalloc(&m->x_base, total) != cudaSuccess) { cudaGetLastError(); m->x_base = nullptr; ok = 0.f; }
    }
    if (ok > 0.f) {
        if (cudaMemsetAsync(m->x_base, 0, total, m->stream) != cudaSuccess || cudaIpcGetMemHandle(&mine, m->x_base) != cudaSuccess) {
            cudaGetLastError();
            ok = 0.f;
        }
    }
    int32_t rc;
    // gather the handles (64 bytes = 16 floats per rank) and a success flag
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
    float* d_buf = nullptr;
    const size_t per = 16 + 1;
    if ((rc = dalloc(m, &d_buf, per * (1 + (size_t)t)))) return rc;
    float h_send[17];
    memcpy(h_send, &mine, 64);
    h_send[16] = ok;
    LTHN_CUDA_TRY(cudaMemcpyAsync(d_buf, h_send, sizeof(h_send), cudaMemcpyHostToDevice, m->stream));
    if ((rc = nccl_check(g_nccl.AllGather(d_buf, d_buf + per, per, kNcclFloat32, m->comm, m->stream), "ncclAllGather"))) return rc;
    std::vector<float> h_all(per * t);
    LTHN_CUDA_TRY(cudaMemcpyAsync(h_all.data(), d_buf + per, per * t * sizeof(float), cudaMemcpyDeviceToHost, m->stream));
    LTHN_CUDA_TRY(cudaStreamSynchronize(m->stream));
    bool all_ok = true;
    for (int r = 0; r < t; r++) all_ok = all_ok && h_all[per * r + 16] > 0.f;
    float mapped = all_ok ? 1.f : 0.f;
    if (all_ok) {
        for (int r = 0; r < t && mapped > 0.f; r++) {
            if (r == c.tp_rank) { m->x_peer[r] = m->x_base; continue; }
            cudaIpcMemHandle_t hd;
            memcpy(&hd, &h_all[per * r], 64);
            if (cudaIpcOpenMemHandle(&m->x_peer[r], hd, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) {
                cudaGetLastError();
                m->x_peer[r] = nullptr;
                mapped = 0.f;
            }
        }
    }
    // second round: did every rank map every peer?
    LTHN_CUDA_TRY(cudaMemcpyAsync(d_buf, &mapped, sizeof(float), cudaMemcpyHostToDevice, m->stream));
    if ((rc = nccl_check(g_nccl.AllGather(d_buf, d_buf + per, 1, kNcclFloat32, m->comm, m->stream), "ncclAllGather"))) return rc;
    LTHN_CUDA_TRY(cudaMemcpyAsync(h_all.data(), d_buf + per, t * sizeof(float), cudaMemcpyDeviceToHost, m->stream));
    LTHN_CUDA_TRY(cudaStreamSynchronize(m->stream));
    for (int r = 0; r < t; r++) all_ok = all_ok && h_all[r] > 0.f;
    if (!all_ok) return LTHN_OK;  // NCCL all-reduce path stays in use
    if ((rc = dalloc(m, &m->x_ctr, 64))) return rc;
    LTHN_CUDA_TRY(cudaMemsetAsync(m->x_ctr, 0, 256, m->stream));
    LTHN_CUDA_TRY(cudaStreamSynchronize(m->stream));
    uint32_t* status = device_status_word();
    if (!status) return fail(LTHN_ERR_CUDA, "model: no device status word");
    for (int site = 0; site < 2; site++) {
        PeerGather& g = m->pg[site];
        g.t = t; g.rank = c.tp_rank;
        g.flag_in = (const uint32_t*)m->x_base;
        g.ctr = m->x_ctr;
        g.status = status;
        for (int r = 0; r < t; r++) {
            g.flag_out[r] = (uint32_t*)m->x_peer[r];
            g.part[r] = (const float*)((const unsigned char*)m->x_peer[r] + flag_bytes + site * site_bytes + r * part_bytes);
            m->x_push[site][r] = (float*)((unsigned char*)m->x_peer[r] + flag_bytes + site * site_bytes + c.tp_rank * part_bytes);
        }
        m->x_part[site] = (float*)((unsigned char*)m->x_base + flag_bytes + site * site_bytes + c.tp_rank * part_bytes);
        m->x_site[site] = (float*)((unsigned char*)m->x_base + flag_bytes + site * site_bytes);
    }
    {
        PairGather& g = m->pairg;
        g.t = t; g.rank = c.tp_rank; g.max_rows = kMaxRows;
        g.flag_in = (const uint32_t*)m->x_base;
        g.ctr = m->x_ctr;
        g.status = status;
        g.pairs_in = (const float*)((const unsigned char*)m->x_base + flag_bytes + 2 * site_bytes);
        for (int r = 0; r < t; r++) {
            g.flag_out[r] = (uint32_t*)m->x_peer[r];
            g.pairs_out[r] = (float*)((unsigned char*)m->x_peer[r] + flag_bytes + 2 * site_bytes);
        }
    }
    m->x_stride = (int64_t)(part_bytes / sizeof(float));
    {
        PeerWait pw{};
        pw.t = t; pw.rank = c.tp_rank; pw.flag_in = (const uint32_t*)m->x_base; pw.ctr = m->x_ctr;
        for (int r = 0; r < t; r++) pw.flag_out[r] = (uint32_t*)m->x_peer[r];
        if ((rc = dalloc(m, &m->d_pw, 1))) return rc;
        LTHN_CUDA_TRY(cudaMemcpy(m->d_pw, &pw, sizeof(pw), cudaMemcpyHostToDevice));
        for (int site = 0; site < 2; site++) {
            if ((rc = dalloc(m, &m->d_push[site], 8))) return rc;
            LTHN_CUDA_TRY(cudaMemcpy(m->d_push[site], m->x_push[site], sizeof(float*) * 8, cudaMemcpyHostToDevice));
        }
    }
    {
        // a site can run in push mode when its projection and the matvecs that consume its norm are
        // all served by the batch-1/2 integer tensor-core kernel
        const char* env = getenv("LTHN_CUDA_NO_NORM_FUSION");
        const bool want_f = !(env && env[0] == '1');
        const Layer& L0 = m->layers[0];
        I8Plan pl;
        m->site_fused[0] = want_f && i8_plan(L0.o.N, L0.o.K, 2, 0, 0, 0, &pl) && qmv_can_fuse_norm(L0.gate.N, L0.gate.K, 2, true);
        m->site_fused[1] = want_f && i8_plan(L0.down.N, L0.down.K, 2, 0, 0, 0, &pl) && qmv_can_fuse_norm(L0.qkv.N, L0.qkv.K, 2, false) &&
                           qmv_can_fuse_norm(m->head.N, m->head.K, 2, false);
    }
    m->xchg_ready = true;
    return LTHN_OK;
}

int32_t lthn_model_finalize(void* model) {
    clear_error();
    Model* m = (Model*)model;
    LTHN_REQUIRE(m != nullptr, "lthn_model_finalize: model is NULL");
    LTHN_REQUIRE(m->have_embed, "lthn_model_finalize: the embedding table was not uploaded");
    for (int li = 0; li < m->c.layers; li++)
        for (int r = 0; r < ROLE_COUNT; r++)
            LTHN_REQUIRE(m->layers[li].have[r], "lthn_model_finalize: a layer is missing a linear");
    if (m->c.tp_size > 1) {
        LTHN_REQUIRE(m->comm != nullptr, "lthn_model_finalize: tensor-parallel model needs a communicator");
        int32_t rc = xchg_setup(m);
        if (rc) return rc;
    }
    {
        const char* env = getenv("LTHN_CUDA_NO_NORM_FUSION");
        const Layer& L0 = m->layers[0];
        m->fuse_norm = !(env && env[0] == '1') && m->c.tp_size <= 1 && qmv_can_fuse_norm(L0.qkv.N, L0.qkv.K, 2, false) &&
                       qmv_can_fuse_norm(L0.gate.N, L0.gate.K, 1, true) && qmv_can_fuse_norm(m->head.N, m->head.K, 2, false);
    }
    if (m->mixed) {
        // 8-bit MLP projections. The norms stay inside the matvecs, and prompts on the prefill GEMM (whose GeGLU
        // tile holds rows of both matrices), when every block's gate/up pair has one width and, where that is 8 bits,
        // the 8-bit matvec plans the fused pair with the norm prologue.
        const Layer& L0 = m->layers[0];
        I8Plan pl;
        m->pair8_ok = i8_plan_b8(L0.gate.N, L0.gate.K, 2, &pl, 0, 0, 1, false);
        bool ok = true, any_pair8 = false;
        for (const Layer& L : m->layers) {
            ok = ok && L.gate.bits == L.up.bits;
            any_pair8 = any_pair8 || L.gate.bits == 8;
        }
        if (any_pair8) ok = ok && m->pair8_ok && qmv_can_fuse_norm(L0.gate.N, L0.gate.K, 2, true, 8);
        m->fuse_norm = m->fuse_norm && ok;
        for (const Layer& L : m->layers) m->prefill_tc = m->prefill_tc && L.gate.bits == L.up.bits;
    }
    {
        // Opt-in (LTHN_CUDA_ATTN_FUSION=1): measured slower than the three kernels it replaces - every CTA repeats the
        // head norms in front of its loads, and the merge by the last CTA puts a fence + counter round trip on the tail.
        const char* env = getenv("LTHN_CUDA_ATTN_FUSION");
        m->attn_fused = env && env[0] == '1' && m->c.sliding_window == 0 && sdpa_fused_supported(m->Hq_l, m->Hkv_l, m->c.head_dim);
        if (m->attn_fused) {
            int32_t rc;
            if ((rc = dalloc(m, &m->att_ctr, (size_t)kMaxRows * m->Hkv_l))) return rc;
            LTHN_CUDA_TRY(cudaMemset(m->att_ctr, 0, (size_t)kMaxRows * m->Hkv_l * sizeof(uint32_t)));
        }
    }
    {
        // the one-kernel decode step serves one row on one GPU, behind the fused final norm of the lm_head
        const auto& c = m->c;
        // Off unless LTHN_CUDA_PERSIST=1: measured slower than the kernel chain on both benchmark models so far.
        const char* env = getenv("LTHN_CUDA_PERSIST");
        std::string why;
        if (env && env[0] == '1' && c.tp_size <= 1 && m->fuse_norm && !m->mixed && c.sliding_window == 0 &&
            persist_supported(c.hidden, m->Hq_l, m->Hkv_l, c.head_dim, m->F_l, &why)) {
            int32_t rc;
            PersistArgs& a = m->pk;
            if ((rc = persist_plan(c.hidden, m->Hq_l, m->Hkv_l, c.head_dim, m->F_l, &a, &m->pk_smem))) return rc;
            std::vector<PersistLayer> pl(c.layers);
            for (int li = 0; li < c.layers; li++) {
                const Layer& L = m->layers[li];
                PersistLayer& d = pl[li];
                d.qkv_w = L.qkv.wq; d.qkv_s = L.qkv.s; d.qkv_b = L.qkv.b;
                d.o_w = L.o.wq; d.o_s = L.o.s; d.o_b = L.o.b;
                d.gate_w = L.gate.wq; d.gate_s = L.gate.s; d.gate_b = L.gate.b;
                d.up_w = L.up.wq; d.up_s = L.up.s; d.up_b = L.up.b;
                d.down_w = L.down.wq; d.down_s = L.down.s; d.down_b = L.down.b;
                d.n_input = L.norm[NORM_INPUT]; d.n_q = L.norm[NORM_Q]; d.n_k = L.norm[NORM_K];
                d.n_post_attn = L.norm[NORM_POST_ATTN]; d.n_pre_ff = L.norm[NORM_PRE_FF]; d.n_post_ff = L.norm[NORM_POST_FF];
                d.kcache = m->kcache + (int64_t)li * m->layer_stride;
                d.vcache = m->vcache + (int64_t)li * m->layer_stride;
            }
            PersistLayer* dl = nullptr;
            if ((rc = dalloc(m, &dl, pl.size()))) return rc;
            LTHN_CUDA_TRY(cudaMemcpy(dl, pl.data(), pl.size() * sizeof(PersistLayer), cudaMemcpyHostToDevice));
            uint32_t* sync = nullptr;
            if ((rc = dalloc(m, &sync, (size_t)PERSIST_SYNC_WORDS))) return rc;
            int chunk_len = 0;
            a.layers = dl; a.nlayers = c.layers;
            a.H = c.hidden; a.Hq = m->Hq_l; a.Hkv = m->Hkv_l; a.D = c.head_dim; a.F = m->F_l;
            a.eps = c.eps; a.attn_scale = c.attn_scale; a.inv_h = 1.0 / (double)c.hidden;
            a.row_pos = m->d_pos; a.row_lane = m->d_lane; a.lane_stride = m->lane_stride; a.max_len = c.max_len;
            a.rope = m->rope;
            a.h0 = m->h; a.h1 = m->h2; a.qkv = m->qkv; a.a = m->a; a.act = m->act; a.part = m->sdpa_part;
            if ((rc = dalloc(m, &a.dig_att, persist_digit_bytes(m->Hq_l, c.head_dim, m->F_l))) ||
                (rc = dalloc(m, &a.dig_act, persist_digit_bytes(m->Hq_l, c.head_dim, m->F_l))))
                return rc;
            a.nchunks_cap = sdpa_item_chunks(c.max_len, c.head_dim);
            a.sync = sync;
            a.status = device_status_word();
            m->persist_ok = true;
        }
    }
    m->finalized = true;
    return LTHN_OK;
}

int32_t lthn_model_weight_bytes(void* model, uint64_t* bytes) {
    clear_error();
    LTHN_REQUIRE(model && bytes, "lthn_model_weight_bytes: NULL argument");
    *bytes = ((Model*)model)->weight_bytes;
    return LTHN_OK;
}

int32_t lthn_model_tp_exchange(void* model, int32_t* mode) {
    clear_error();
    Model* m = (Model*)model;
    LTHN_REQUIRE(m && mode, "lthn_model_tp_exchange: NULL argument");
    LTHN_REQUIRE(m->finalized, "lthn_model_tp_exchange: model is not finalized");
    *mode = m->c.tp_size <= 1 ? 0 : (m->xchg_ready ? 2 : 1);
    return LTHN_OK;
}

int32_t lthn_model_decode_kernel(void* model, int32_t* mode) {
    clear_error();
    Model* m = (Model*)model;
    LTHN_REQUIRE(m && mode, "lthn_model_decode_kernel: NULL argument");
    LTHN_REQUIRE(m->finalized, "lthn_model_decode_kernel: model is not finalized");
    *mode = m->persist_ok ? 1 : 0;
    return LTHN_OK;
}

// 0: decode steps have not been captured (yet), 1: they replay a CUDA graph, 2: capture was not
// possible and steps are launched kernel by kernel
int32_t lthn_model_graph_state(void* model, int32_t* state) {
    clear_error();
    Model* m = (Model*)model;
    LTHN_REQUIRE(m && state, "lthn_model_graph_state: NULL argument");
    *state = m->graphs_off ? 2 : 0;
    for (auto g : m->step_graph) if (g) *state = 1;
    return LTHN_OK;
}

int32_t lthn_model_destroy(void* model) {
    clear_error();
    Model* m = (Model*)model;
    if (!m) return LTHN_OK;
    cudaStreamSynchronize(m->stream);
    for (auto& g : m->step_graph)
        if (g) cudaGraphExecDestroy(g);
    for (auto e : m->trace.ev) cudaEventDestroy(e);
    for (int r = 0; r < 8; r++)
        if (m->x_peer[r] && m->x_peer[r] != m->x_base) cudaIpcCloseMemHandle(m->x_peer[r]);
    if (m->x_base) cudaFree(m->x_base);
    for (void* p : m->allocs) cudaFree(p);
    if (m->h_pinned) cudaFreeHost(m->h_pinned);
    if (m->p_pinned) cudaFreeHost(m->p_pinned);
    cudaStreamDestroy(m->stream);
    delete m;
    return LTHN_OK;
}

// ---- session ------------------------------------------------------------------------------------
int32_t lthn_session_open(void* model, void** session) {
    clear_error();
    Model* m = (Model*)model;
    LTHN_REQUIRE(m && session, "lthn_session_open: NULL argument");
    LTHN_REQUIRE(m->finalized, "lthn_session_open: model is not finalized");
    const int id = lane_acquire(m);
    if (id < 0) return fail(LTHN_ERR_STATE, "lthn_session_open: every KV lane is in use");
    Session* s = new Session{m, Lane{}};
    s->lane.id = id;
    *session = s;
    return LTHN_OK;
}

int32_t lthn_session_close(void* session) {
    clear_error();
    Session* s = (Session*)session;
    if (!s) return LTHN_OK;
    lane_release(s->m, s->lane.id);
    delete s;
    return LTHN_OK;
}

int32_t lthn_session_prefill(void* session, const int32_t* ids, int32_t n) {
    clear_error();
    Session* s = (Session*)session;
    LTHN_REQUIRE(s && ids, "lthn_session_prefill: NULL argument");
    s->lane.pos = 0;
    s->lane.pending = -1;
    s->lane.have_next = false;
    return feed_lane(s->m, &s->lane, ids, n);
}

int32_t lthn_session_append(void* session, const int32_t* ids, int32_t n) {
    clear_error();
    Session* s = (Session*)session;
    LTHN_REQUIRE(s && ids, "lthn_session_append: NULL argument");
    if (s->lane.pending >= 0) {  // a generated token that was yielded but not yet fed comes first
        const int32_t t = s->lane.pending;
        int32_t rc = feed_lane(s->m, &s->lane, &t, 1);
        if (rc) return rc;
    }
    return feed_lane(s->m, &s->lane, ids, n);
}

int32_t lthn_session_pos(void* session) {
    Session* s = (Session*)session;
    return s ? s->lane.pos : -1;
}

// GenerateFromCacheEach (engine/session.go:49): up to max_new greedy tokens; eos_id < 0
// leaves the stop decision to the caller. The last produced token is not fed.
int32_t lthn_session_decode_greedy(void* session, int32_t max_new, int32_t eos_id, int32_t* out_ids, int32_t* n_out) {
    clear_error();
    Session* s = (Session*)session;
    LTHN_REQUIRE(s && out_ids && n_out, "lthn_session_decode_greedy: NULL argument");
    *n_out = 0;
    LTHN_REQUIRE(s->lane.pos > 0, "lthn_session_decode_greedy: the session has no prefilled state");
    for (int i = 0; i < max_new; i++) {
        if (!s->lane.have_next) {
            LTHN_REQUIRE(s->lane.pending >= 0, "lthn_session_decode_greedy: no pending token");
            if (s->lane.pos + 1 > s->m->c.max_len) return fail(LTHN_ERR_STATE, "lthn_session_decode_greedy: context length exceeded");
            const int32_t t = s->lane.pending;
            int32_t rc = feed_lane(s->m, &s->lane, &t, 1);
            if (rc) return rc;
        }
        const int32_t tok = s->lane.next_tok;
        out_ids[(*n_out)++] = tok;
        s->lane.pending = tok;
        s->lane.have_next = false;
        if (eos_id >= 0 && tok == eos_id) break;
    }
    return LTHN_OK;
}

// engine.DecodePhaseTracer.BeginDecodePhaseTrace (engine/session.go:86-98): phase timing for the one-row decode
// steps that follow on this session's model, until lthn_session_trace_end returns the aggregate
// (inference.DecodePhaseBudget, inference.go:218-268). A single-flight diagnostic, as in the reference:
// while it is on, steps are launched kernel by kernel (no graph replay) with an event between phases.
int32_t lthn_session_trace_begin(void* session) {
    clear_error();
    Session* s = (Session*)session;
    LTHN_REQUIRE(s != nullptr, "lthn_session_trace_begin: NULL argument");
    Model* m = s->m;
    std::lock_guard<std::mutex> lk(m->mu);
    auto& t = m->trace;
    t.on = true;
    t.used = 0;
    t.tokens = 0;
    t.gpu_us = 0;
    for (double& p : t.phase_us) p = 0;
    t.t0 = std::chrono::steady_clock::now();
    return LTHN_OK;
}

int32_t lthn_session_trace_end(void* session, lthn_decode_phase_budget* out) {
    clear_error();
    Session* s = (Session*)session;
    LTHN_REQUIRE(s && out, "lthn_session_trace_end: NULL argument");
    Model* m = s->m;
    std::lock_guard<std::mutex> lk(m->mu);
    auto& t = m->trace;
    memset(out, 0, sizeof(*out));
    if (!t.on || t.tokens <= 0) { t.on = false; return LTHN_OK; }  // nothing traced: a zero budget, as the reference returns
    const double wall_us = std::chrono::duration<double, std::micro>(std::chrono::steady_clock::now() - t.t0).count();
    t.on = false;
    out->tokens = t.tokens;
    out->total_per_token_us = wall_us / t.tokens;
    out->gpu_per_token_us = t.gpu_us / t.tokens;
    for (int p = 0; p < PH_COUNT; p++) {
        if (t.phase_us[p] <= 0) continue;
        auto& ph = out->phases[out->n_phases++];
        snprintf(ph.name, sizeof(ph.name), "%s", kPhaseName[p]);
        ph.per_token_us = t.phase_us[p] / t.tokens;
        ph.gpu = 1;
    }
    return LTHN_OK;
}

// GenerateSampledFromCacheEach (engine/session.go:51): the loop of model/token.go:263-305 with the
// pick made by the sampler. The repeat-penalty history is the tokens of this call.
int32_t lthn_session_decode_sampled(void* session, void* sampler, const lthn_sample_params* params, int32_t max_new,
                                    const int32_t* stop, int32_t n_stop, int32_t* out_ids, int32_t* n_out) {
    clear_error();
    Session* s = (Session*)session;
    LTHN_REQUIRE(s && sampler && params && out_ids && n_out, "lthn_session_decode_sampled: NULL argument");
    LTHN_REQUIRE(n_stop >= 0 && (n_stop == 0 || stop), "lthn_session_decode_sampled: bad stop list");
    LTHN_REQUIRE(params->n_suppress >= 0 && (params->n_suppress == 0 || params->suppress), "lthn_session_decode_sampled: bad suppress list");
    *n_out = 0;
    LTHN_REQUIRE(s->lane.pos > 0, "lthn_session_decode_sampled: the session has no prefilled state");
    Model* m = s->m;
    SampleState st;
    st.rng = (HostSampler*)sampler;
    st.p = *params;
    if (params->n_suppress) st.suppress.assign(params->suppress, params->suppress + params->n_suppress);
    const std::vector<int32_t> stops(stop, stop + n_stop);
    for (int i = 0; i < max_new; i++) {
        if (!s->lane.have_next) {  // the last picked token has not been fed yet: its logits are needed now
            LTHN_REQUIRE(s->lane.pending >= 0, "lthn_session_decode_sampled: no pending token");
            if (s->lane.pos + 1 > m->c.max_len) return fail(LTHN_ERR_STATE, "lthn_session_decode_sampled: context length exceeded");
            const int32_t t = s->lane.pending;
            int32_t rc = feed_lane(m, &s->lane, &t, 1);
            if (rc) return rc;
        }
        int32_t tok = -1;
        {
            std::lock_guard<std::mutex> lk(m->mu);
            if (s->lane.logits_serial != m->logits_serial)
                return fail(LTHN_ERR_STATE, "lthn_session_decode_sampled: a later forward of another session or lane set of this model has "
                                            "overwritten the logits");
            int32_t rc = sample_row(m, s->lane.logits_row, st, stops, &tok);
            if (rc) return rc;
        }
        out_ids[(*n_out)++] = tok;
        st.generated++;
        if (st.p.repeat_penalty > 1.0f) st.history.push_back(tok);
        s->lane.pending = tok;
        s->lane.have_next = false;
        if (std::find(stops.begin(), stops.end(), tok) != stops.end()) break;
    }
    return LTHN_OK;
}

// Logits of the last fed token (vocab floats; local shard under tensor parallelism) for
// host-side sampling (engine/session.go:51 GenerateSampledFromCacheEach).
int32_t lthn_session_logits(void* session, float* logits_host, int64_t n) {
    clear_error();
    Session* s = (Session*)session;
    LTHN_REQUIRE(s && logits_host, "lthn_session_logits: NULL argument");
    LTHN_REQUIRE(s->lane.have_next, "lthn_session_logits: no forward has been run since the last token was taken");
    LTHN_REQUIRE(n == s->m->V_l, "lthn_session_logits: buffer must hold the (local) vocabulary");
    std::lock_guard<std::mutex> lk(s->m->mu);
    if (s->lane.logits_serial != s->m->logits_serial)
        return fail(LTHN_ERR_STATE, "lthn_session_logits: a later forward of another session or lane set of this model has "
                                    "overwritten the logits; read them before the next forward on the model");
    LTHN_CUDA_TRY(cudaMemcpyAsync(logits_host, s->m->logits + (size_t)s->lane.logits_row * n, (size_t)n * 4, cudaMemcpyDeviceToHost, s->m->stream));
    LTHN_CUDA_TRY(cudaStreamSynchronize(s->m->stream));
    return LTHN_OK;
}

// KV read-out of one layer (bf16 [pos, kv_heads_local*head_dim]) - the payload of a
// kv.Snapshot layer (kv/snapshot.go:98-143); which: 0 keys, 1 values.
int32_t lthn_session_kv_export(void* session, int32_t layer, int32_t which, void* out_host, size_t out_bytes) {
    clear_error();
    Session* s = (Session*)session;
    LTHN_REQUIRE(s && out_host, "lthn_session_kv_export: NULL argument");
    Model* m = s->m;
    LTHN_REQUIRE(layer >= 0 && layer < m->c.layers, "lthn_session_kv_export: layer out of range");
    const size_t bytes = (size_t)s->lane.pos * m->KR_l * 2;
    LTHN_REQUIRE(out_bytes == bytes, "lthn_session_kv_export: buffer must hold pos*kv_heads*head_dim bf16 values");
    const uint16_t* src = (which ? m->vcache : m->kcache) + (int64_t)s->lane.id * m->lane_stride + (int64_t)layer * m->layer_stride;
    std::lock_guard<std::mutex> lk(m->mu);
    LTHN_CUDA_TRY(cudaMemcpyAsync(out_host, src, bytes, cudaMemcpyDeviceToHost, m->stream));
    LTHN_CUDA_TRY(cudaStreamSynchronize(m->stream));
    return LTHN_OK;
}

int32_t lthn_session_kv_import(void* session, int32_t layer, int32_t which, const void* in_host, int32_t tokens) {
    clear_error();
    Session* s = (Session*)session;
    LTHN_REQUIRE(s && in_host, "lthn_session_kv_import: NULL argument");
    Model* m = s->m;
    LTHN_REQUIRE(layer >= 0 && layer < m->c.layers && tokens >= 0 && tokens <= m->c.max_len, "lthn_session_kv_import: out of range");
    uint16_t* dst = (which ? m->vcache : m->kcache) + (int64_t)s->lane.id * m->lane_stride + (int64_t)layer * m->layer_stride;
    std::lock_guard<std::mutex> lk(m->mu);
    LTHN_CUDA_TRY(cudaMemcpyAsync(dst, in_host, (size_t)tokens * m->KR_l * 2, cudaMemcpyHostToDevice, m->stream));
    LTHN_CUDA_TRY(cudaStreamSynchronize(m->stream));
    return LTHN_OK;
}

// kv.Snapshot support (kv/snapshot.go:98-143, engine/session.go:53-58): token ranges of a layer's cache -
// what RangeKVBlocks streams block by block and CaptureOptions.BlockStartToken skips a prefix of.
static int32_t kv_range_check(Session* s, int32_t layer, int32_t token0, int32_t ntokens, bool within_pos, const char* who) {
    Model* m = s->m;
    if (layer < 0 || layer >= m->c.layers) return fail(LTHN_ERR_INVALID, std::string(who) + ": layer out of range");
    if (token0 < 0 || ntokens < 0 || (int64_t)token0 + ntokens > (within_pos ? s->lane.pos : m->c.max_len))
        return fail(LTHN_ERR_INVALID, std::string(who) + (within_pos ? ": token range reaches past the session's position" : ": token range reaches past the context length"));
    return LTHN_OK;
}

int32_t lthn_session_kv_export_range(void* session, int32_t layer, int32_t which, int32_t token0, int32_t ntokens, void* out_host,
                                     size_t out_bytes) {
    clear_error();
    Session* s = (Session*)session;
    LTHN_REQUIRE(s && (out_host || ntokens == 0), "lthn_session_kv_export_range: NULL argument");
    int32_t rc;
    if ((rc = kv_range_check(s, layer, token0, ntokens, true, "lthn_session_kv_export_range"))) return rc;
    Model* m = s->m;
    const size_t bytes = (size_t)ntokens * m->KR_l * 2;
    LTHN_REQUIRE(out_bytes == bytes, "lthn_session_kv_export_range: buffer must hold ntokens*kv_heads*head_dim bf16 values");
    if (!bytes) return LTHN_OK;
    const uint16_t* src = (which ? m->vcache : m->kcache) + (int64_t)s->lane.id * m->lane_stride + (int64_t)layer * m->layer_stride +
                          (int64_t)token0 * m->KR_l;
    std::lock_guard<std::mutex> lk(m->mu);
    LTHN_CUDA_TRY(cudaMemcpyAsync(out_host, src, bytes, cudaMemcpyDeviceToHost, m->stream));
    LTHN_CUDA_TRY(cudaStreamSynchronize(m->stream));
    return LTHN_OK;
}

int32_t lthn_session_kv_import_range(void* session, int32_t layer, int32_t which, int32_t token0, const void* in_host, int32_t ntokens) {
    clear_error();
    Session* s = (Session*)session;
    LTHN_REQUIRE(s && (in_host || ntokens == 0), "lthn_session_kv_import_range: NULL argument");
    int32_t rc;
    if ((rc = kv_range_check(s, layer, token0, ntokens, false, "lthn_session_kv_import_range"))) return rc;
    if (!ntokens) return LTHN_OK;
    Model* m = s->m;
    uint16_t* dst = (which ? m->vcache : m->kcache) + (int64_t)s->lane.id * m->lane_stride + (int64_t)layer * m->layer_stride +
                    (int64_t)token0 * m->KR_l;
    std::lock_guard<std::mutex> lk(m->mu);
    LTHN_CUDA_TRY(cudaMemcpyAsync(dst, in_host, (size_t)ntokens * m->KR_l * 2, cudaMemcpyHostToDevice, m->stream));
    LTHN_CUDA_TRY(cudaStreamSynchronize(m->stream));
    return LTHN_OK;
}

// Under tensor parallelism a rank holds kv_heads/tp of the heads. Every rank calls this with the same
// arguments; each gets the rows with all heads in model order ([ntokens][kv_heads*head_dim]), gathered
// with one NCCL all-gather. On a single GPU it is lthn_session_kv_export_range.
int32_t lthn_session_kv_gather_range(void* session, int32_t layer, int32_t which, int32_t token0, int32_t ntokens, void* out_host,
                                     size_t out_bytes) {
    clear_error();
    Session* s = (Session*)session;
    LTHN_REQUIRE(s && (out_host || ntokens == 0), "lthn_session_kv_gather_range: NULL argument");
    Model* m = s->m;
    const int t = std::max(1, m->c.tp_size);
    if (t == 1) return lthn_session_kv_export_range(session, layer, which, token0, ntokens, out_host, out_bytes);
    int32_t rc;
    if ((rc = kv_range_check(s, layer, token0, ntokens, true, "lthn_session_kv_gather_range"))) return rc;
    const size_t per = (size_t)ntokens * m->KR_l * 2;  // bytes of one rank's rows
    LTHN_REQUIRE(out_bytes == per * t, "lthn_session_kv_gather_range: buffer must hold ntokens*kv_heads*head_dim bf16 values of the whole model");
    if (!per) return LTHN_OK;
    if (!m->comm) return fail(LTHN_ERR_STATE, "lthn_session_kv_gather_range: the model has no communicator");
    void* scratch = nullptr;
    if ((rc = scratch_get(per * t, &scratch, 3))) return rc;
    const uint16_t* src = (which ? m->vcache : m->kcache) + (int64_t)s->lane.id * m->lane_stride + (int64_t)layer * m->layer_stride +
                          (int64_t)token0 * m->KR_l;
    std::vector<uint16_t> all(per * t / 2);
    {
        std::lock_guard<std::mutex> lk(m->mu);
        if ((rc = nccl_check(g_nccl.AllGather(src, scratch, per / 4, kNcclFloat32, m->comm, m->stream), "ncclAllGather"))) return rc;
        LTHN_CUDA_TRY(cudaMemcpyAsync(all.data(), scratch, per * t, cudaMemcpyDeviceToHost, m->stream));
        LTHN_CUDA_TRY(cudaStreamSynchronize(m->stream));
    }
    // [rank][token][local heads] -> [token][rank][local heads]
    uint16_t* out = (uint16_t*)out_host;
    const size_t kr = (size_t)m->KR_l;
    for (int r = 0; r < t; r++)
        for (int tk = 0; tk < ntokens; tk++)
            memcpy(out + ((size_t)tk * t + r) * kr, all.data() + ((size_t)r * ntokens + tk) * kr, kr * 2);
    return LTHN_OK;
}

// Session.Fork (enginetest/session.go:72-90): a second session on a KV lane of its own that starts as a
// copy of this one - the cache rows up to the position are copied on the device - and then advances
// independently.
int32_t lthn_session_fork(void* session, void** fork) {
    clear_error();
    Session* s = (Session*)session;
    LTHN_REQUIRE(s && fork, "lthn_session_fork: NULL argument");
    Model* m = s->m;
    const int id = lane_acquire(m);
    if (id < 0) return fail(LTHN_ERR_STATE, "lthn_session_fork: every KV lane is in use");
    Session* f = new Session{m, s->lane};
    f->lane.id = id;
    f->lane.logits_serial = 0;  // the fork has no logits of its own: the model's buffer belongs to the parent's last forward
    f->lane.samp.reset();
    {
        std::lock_guard<std::mutex> lk(m->mu);
        const size_t bytes = (size_t)s->lane.pos * m->KR_l * 2;
        for (int li = 0; li < m->c.layers && bytes; li++)
            for (int which = 0; which < 2; which++) {
                uint16_t* base = (which ? m->vcache : m->kcache) + (int64_t)li * m->layer_stride;
                const cudaError_t e = cudaMemcpyAsync(base + (int64_t)id * m->lane_stride, base + (int64_t)s->lane.id * m->lane_stride, bytes,
                                                      cudaMemcpyDeviceToDevice, m->stream);
                if (e != cudaSuccess) { lane_release(m, id); delete f; return cuda_fail(e, "cudaMemcpyAsync"); }
            }
        const cudaError_t e = cudaStreamSynchronize(m->stream);
        if (e != cudaSuccess) { lane_release(m, id); delete f; return cuda_fail(e, "cudaStreamSynchronize"); }
    }
    *fork = f;
    return LTHN_OK;
}

// Session.Reset: forget the sequence; the lane stays with the session.
int32_t lthn_session_reset(void* session) {
    clear_error();
    Session* s = (Session*)session;
    LTHN_REQUIRE(s != nullptr, "lthn_session_reset: NULL argument");
    const int id = s->lane.id;
    s->lane = Lane{};
    s->lane.id = id;
    return LTHN_OK;
}

// After importing every layer: declares the restored length and the token to continue from.
int32_t lthn_session_set_state(void* session, int32_t pos, int32_t pending_token) {
    clear_error();
    Session* s = (Session*)session;
    LTHN_REQUIRE(s != nullptr, "lthn_session_set_state: NULL argument");
    LTHN_REQUIRE(pos >= 0 && pos <= s->m->c.max_len, "lthn_session_set_state: pos out of range");
    s->lane.pos = pos;
    s->lane.pending = pending_token;
    s->lane.have_next = false;
    return LTHN_OK;
}

// ---- lane set -------------------------------------------------------------------------------------
int32_t lthn_laneset_open(void* model, int32_t max_lanes, void** set) {
    clear_error();
    Model* m = (Model*)model;
    LTHN_REQUIRE(m && set, "lthn_laneset_open: NULL argument");
    LTHN_REQUIRE(m->finalized, "lthn_laneset_open: model is not finalized");
    if (max_lanes <= 0) max_lanes = std::min(8, m->c.max_lanes);  // cf. hip_lane_set.go:14-16 default of 8
    LTHN_REQUIRE(max_lanes <= kMaxRows, "lthn_laneset_open: at most 32 lanes per set");
    LaneSet* ls = new LaneSet{m, max_lanes, {}, 1, 0};
    *set = ls;
    return LTHN_OK;
}

static int32_t laneset_prepare(LaneSet* ls, const int32_t* ids, int32_t n, int32_t max_new, const int32_t* stop, int32_t n_stop,
                               const lthn_sample_params* params, uint64_t seed, int32_t* lane_handle) {
    LTHN_REQUIRE(ls && ids && lane_handle, "lthn_laneset_prepare: NULL argument");
    LTHN_REQUIRE((int)ls->lanes.size() < ls->max_lanes, "lthn_laneset_prepare: the lane set is at MaxLanes");
    LTHN_REQUIRE(!params || (params->n_suppress >= 0 && (params->n_suppress == 0 || params->suppress)), "lthn_laneset_prepare: bad suppress list");
    const int id = lane_acquire(ls->m);
    if (id < 0) return fail(LTHN_ERR_STATE, "lthn_laneset_prepare: every KV lane of the model is in use");
    Lane ln;
    ln.id = id;
    ln.max_new = max_new;
    if (stop && n_stop > 0) ln.stop.assign(stop, stop + n_stop);
    int32_t rc = feed_lane(ls->m, &ln, ids, n);
    if (rc) { lane_release(ls->m, id); return rc; }
    if (params) {
        // the lane's own sampler state; its first token is drawn now, from the prompt's logits,
        // before another lane's forward overwrites the model's logits buffer
        ln.samp = std::make_shared<SampleState>();
        ln.samp->own.state = seed;
        ln.samp->rng = &ln.samp->own;
        ln.samp->p = *params;
        if (params->n_suppress) ln.samp->suppress.assign(params->suppress, params->suppress + params->n_suppress);
        std::lock_guard<std::mutex> lk(ls->m->mu);
        int32_t tok = -1;
        if ((rc = sample_row(ls->m, ln.logits_row, *ln.samp, ln.stop, &tok))) { lane_release(ls->m, id); return rc; }
        ln.next_tok = tok;
        ln.samp->generated++;
        if (params->repeat_penalty > 1.0f) ln.samp->history.push_back(tok);
    }
    ln.handle = ls->next_handle++;
    ls->lanes.push_back(ln);
    *lane_handle = ln.handle;
    return LTHN_OK;
}

int32_t lthn_laneset_prepare(void* set, const int32_t* ids, int32_t n, int32_t max_new, const int32_t* stop,
                             int32_t n_stop, int32_t* lane_handle) {
    clear_error();
    return laneset_prepare((LaneSet*)set, ids, n, max_new, stop, n_stop, nullptr, 0, lane_handle);
}

int32_t lthn_laneset_prepare_sampled(void* set, const int32_t* ids, int32_t n, int32_t max_new, const int32_t* stop,
                                     int32_t n_stop, const lthn_sample_params* params, uint64_t seed, int32_t* lane_handle) {
    clear_error();
    LTHN_REQUIRE(params != nullptr, "lthn_laneset_prepare_sampled: params is NULL");
    return laneset_prepare((LaneSet*)set, ids, n, max_new, stop, n_stop, params, seed, lane_handle);
}

// One batched forward for every active, non-terminal lane (inference.LaneSet.Step).
// flags: bit0 HasToken, bit1 Terminal. The first Step after Prepare yields the token the
// prefill already determined; every Step runs exactly one forward when any lane has a
// pending token to feed.
int32_t lthn_laneset_step(void* set, int32_t* lane_handles, int32_t* tokens, int32_t* flags, int32_t* n) {
    clear_error();
    LaneSet* ls = (LaneSet*)set;
    LTHN_REQUIRE(ls && lane_handles && tokens && flags && n, "lthn_laneset_step: NULL argument");
    Model* m = ls->m;
    *n = 0;
    std::vector<Lane*> feed;
    for (auto& ln : ls->lanes)
        if (!ln.terminal && !ln.have_next && ln.pending >= 0) feed.push_back(&ln);
    if (!feed.empty()) {
        std::lock_guard<std::mutex> lk(m->mu);
        const int rows = (int)feed.size();
        int32_t* hp = m->h_pinned;
        int max_ctx = 1;
        for (int r = 0; r < rows; r++) {
            if (feed[r]->pos + 1 > m->c.max_len) return fail(LTHN_ERR_STATE, "lthn_laneset_step: context length exceeded");
            hp[r] = feed[r]->pending; hp[kMaxRows + r] = feed[r]->pos; hp[2 * kMaxRows + r] = feed[r]->id;
            max_ctx = std::max(max_ctx, feed[r]->pos + 1);
        }
        LTHN_CUDA_TRY(cudaMemcpyAsync(m->d_ids, hp, 3 * kMaxRows * 4, cudaMemcpyHostToDevice, m->stream));
        int32_t rc = decode_step(m, rows);
        if (rc) return rc;
        LTHN_CUDA_TRY(cudaMemcpyAsync(hp + 3 * kMaxRows, m->d_next, rows * 4, cudaMemcpyDeviceToHost, m->stream));
        if ((rc = device_status_read_async(m->stream, (uint32_t*)(hp + 4 * kMaxRows)))) return rc;
        LTHN_CUDA_TRY(cudaStreamSynchronize(m->stream));
        ++m->logits_serial;
        for (int r = 0; r < rows; r++) {
            feed[r]->pos += 1;
            feed[r]->next_tok = hp[3 * kMaxRows + r];
            feed[r]->have_next = true;
            feed[r]->pending = -1;
            feed[r]->logits_serial = m->logits_serial;
            feed[r]->logits_row = r;
        }
        ls->forwards++;
        trace_collect(m);
        if ((rc = device_status_judge((uint32_t)hp[4 * kMaxRows], m->stream))) return rc;
        // lanes with a sampler draw their token from their row of this forward's logits
        for (int r = 0; r < rows; r++) {
            if (!feed[r]->samp) continue;
            SampleState& st = *feed[r]->samp;
            st.rng = &st.own;
            int32_t tok = -1;
            if ((rc = sample_row(m, r, st, feed[r]->stop, &tok))) return rc;
            feed[r]->next_tok = tok;
            st.generated++;
            if (st.p.repeat_penalty > 1.0f) st.history.push_back(tok);
        }
    }
    for (auto& ln : ls->lanes) {
        if (ln.terminal || !ln.have_next) continue;
        const int32_t tok = ln.next_tok;
        ln.have_next = false;
        ln.pending = tok;
        ln.produced++;
        bool stop = ln.max_new > 0 && ln.produced >= ln.max_new;
        for (int32_t st : ln.stop) stop = stop || st == tok;
        ln.terminal = stop;
        lane_handles[*n] = ln.handle;
        tokens[*n] = tok;
        flags[*n] = 1 | (stop ? 2 : 0);
        (*n)++;
    }
    return LTHN_OK;
}

int32_t lthn_laneset_retire(void* set, int32_t lane_handle) {
    clear_error();
    LaneSet* ls = (LaneSet*)set;
    LTHN_REQUIRE(ls != nullptr, "lthn_laneset_retire: NULL argument");
    for (size_t i = 0; i < ls->lanes.size(); i++)
        if (ls->lanes[i].handle == lane_handle) {
            lane_release(ls->m, ls->lanes[i].id);
            ls->lanes.erase(ls->lanes.begin() + i);
            return LTHN_OK;
        }
    return fail(LTHN_ERR_INVALID, "lthn_laneset_retire: unknown lane");
}

int32_t lthn_laneset_active(void* set) { return set ? (int32_t)((LaneSet*)set)->lanes.size() : 0; }
uint64_t lthn_laneset_batch_forward_count(void* set) { return set ? ((LaneSet*)set)->forwards : 0; }

int32_t lthn_laneset_close(void* set) {
    clear_error();
    LaneSet* ls = (LaneSet*)set;
    if (!ls) return LTHN_OK;
    for (auto& ln : ls->lanes) lane_release(ls->m, ln.id);
    delete ls;
    return LTHN_OK;
}

// ---- standalone fused kernels (for callers that drive the layer loop themselves) -----------------
int32_t lthn_rmsnorm(void* stream, const float* x, const float* w, float* out, int32_t rows, int32_t width, float eps) {
    clear_error();
    if (rows == 0) return LTHN_OK;
    LTHN_REQUIRE(x && w && out && rows > 0 && width > 0 && eps >= 0, "lthn_rmsnorm: bad arguments");
    return launch_rmsnorm((cudaStream_t)stream, x, nullptr, w, nullptr, out, rows, width, eps, 0);
}

int32_t lthn_rmsnorm_residual(void* stream, const float* a, float* h, const float* w_post, const float* w_next,
                              float* out, int32_t rows, int32_t width, float eps) {
    clear_error();
    if (rows == 0) return LTHN_OK;
    LTHN_REQUIRE(a && h && w_post && w_next && out && rows > 0 && width > 0 && eps >= 0, "lthn_rmsnorm_residual: bad arguments");
    return launch_rmsnorm((cudaStream_t)stream, a, h, w_post, w_next, out, rows, width, eps, 1);
}

int32_t lthn_rmsnorm_rope(void* stream, const float* x, const float* w, const int32_t* positions, float* out,
                          int32_t rows, int32_t heads, int32_t head_dim, int32_t rotary_dim, float eps, float rope_base,
                          int32_t bf16_seams) {
    clear_error();
    if (rows == 0 || heads == 0) return LTHN_OK;
    LTHN_REQUIRE(x && w && positions && out && rows > 0 && heads > 0, "lthn_rmsnorm_rope: bad arguments");
    LTHN_REQUIRE(head_dim > 0 && head_dim <= 512 && head_dim % 64 == 0, "lthn_rmsnorm_rope: head_dim must be a multiple of 64 up to 512");
    if (rotary_dim == 0) rotary_dim = head_dim;
    LTHN_REQUIRE(rotary_dim > 0 && rotary_dim <= head_dim && rotary_dim % 2 == 0, "lthn_rmsnorm_rope: rotary_dim must be even and at most head_dim");
    LTHN_REQUIRE(rope_base > 0 && eps >= 0, "lthn_rmsnorm_rope: base must be positive and eps non-negative");
    return launch_rmsnorm_rope((cudaStream_t)stream, x, w, positions, out, rows, heads, head_dim, rotary_dim, eps, rope_base, bf16_seams);
}

int32_t lthn_sdpa_decode(void* stream, const float* q, const uint16_t* kcache, const uint16_t* vcache,
                         const int32_t* row_pos, const int32_t* row_lane, float* out, int32_t rows, int32_t q_heads,
                         int32_t kv_heads, int32_t head_dim, int64_t lane_stride, float scale, int32_t max_ctx) {
    clear_error();
    if (rows == 0) return LTHN_OK;
    LTHN_REQUIRE(q && kcache && vcache && row_pos && row_lane && out, "lthn_sdpa_decode: NULL pointer");
    LTHN_REQUIRE(rows > 0 && q_heads > 0 && kv_heads > 0 && max_ctx > 0, "lthn_sdpa_decode: dimensions must be positive");
    if (scale <= 0) scale = (float)(1.0 / std::sqrt((double)head_dim));
    int chunk_len = 0;
    const int nchunks = sdpa_chunking(max_ctx, head_dim, &chunk_len, rows, std::max(1, kv_heads));
    void* part = nullptr;
    if (nchunks > 1) {
        int32_t rc = scratch_get(sdpa_scratch_bytes(rows, q_heads, head_dim, nchunks), &part, 2);
        if (rc) return rc;
    }
    SdpaArgs a{q, kcache, vcache, row_pos, row_lane, out, (float*)part, lane_stride, q_heads, kv_heads, nchunks, chunk_len, scale};
    return launch_sdpa_decode((cudaStream_t)stream, a, rows, head_dim);
}

int32_t lthn_prefill_attention(void* stream, const float* q, const uint16_t* kcache, const uint16_t* vcache, uint16_t* out,
                               int32_t rows, int32_t pos0, int32_t q_heads, int32_t kv_heads, int32_t head_dim, float scale) {
    clear_error();
    if (rows == 0) return LTHN_OK;
    LTHN_REQUIRE(q && kcache && vcache && out, "lthn_prefill_attention: NULL pointer");
    LTHN_REQUIRE(rows > 0 && pos0 >= 0 && q_heads > 0 && kv_heads > 0, "lthn_prefill_attention: dimensions must be positive");
    LTHN_REQUIRE((((uintptr_t)q | (uintptr_t)kcache | (uintptr_t)vcache) & 15) == 0 && ((uintptr_t)out & 3) == 0,
                 "lthn_prefill_attention: q and the caches must be 16-byte aligned");
    if (scale <= 0) scale = (float)(1.0 / std::sqrt((double)head_dim));
    PrefillAttnArgs a{q, kcache, vcache, out, rows, pos0, q_heads, kv_heads, (float)((double)scale * 1.4426950408889634)};
    return launch_prefill_attn((cudaStream_t)stream, a, head_dim);
}

int32_t lthn_argmax(void* stream, const float* logits, int32_t rows, int32_t vocab, int32_t* out_idx) {
    clear_error();
    if (rows == 0) return LTHN_OK;
    LTHN_REQUIRE(logits && out_idx && rows > 0 && vocab > 0, "lthn_argmax: bad arguments");
    void* scratch = nullptr;
    int32_t rc = scratch_get((size_t)rows * ARGMAX_BLOCKS * 8, &scratch, 3);
    if (rc) return rc;
    float* pv = (float*)scratch;
    int* pi = (int*)(pv + (size_t)rows * ARGMAX_BLOCKS);
    return launch_argmax((cudaStream_t)stream, logits, rows, vocab, pv, pi, out_idx, nullptr, 0);
}

}  // extern "C"
