/*
 * lthn_cuda.h — C ABI of liblthn_cuda.so, the B200 (sm_100a) engine for
 * go-inference's MLX-affine quantized-linear hot path.
 *
 * This is the surface a cgo shim in a Go package `engine/cuda` binds. Every
 * function returns an int32 status (0 = LTHN_OK); on failure a message is kept
 * per calling thread and read with lthn_last_error(). Nothing throws, nothing
 * calls back into the host language, and no host pointer is retained after a
 * call returns. Device pointers are plain `void*`; streams are `void*` holding a
 * cudaStream_t (NULL = the legacy default stream).
 *
 * Reference citations give the file:line of the go-inference interface each
 * entry point stands behind (paths relative to the reference's `go/` directory).
 *
 * Weight layout everywhere (go/model/quant/mlxaffine/mlxaffine.go:14-21):
 *   packed  uint32 [N, K*bits/32], code p of a word at bits [p*bits, p*bits+bits)
 *   scales  bf16   [N, K/group_size]
 *   biases  bf16   [N, K/group_size]
 *   w[n,k] = scale[n,k/gs] * code + bias[n,k/gs]
 */
#ifndef LTHN_CUDA_H
#define LTHN_CUDA_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum {
    LTHN_OK = 0,
    LTHN_ERR_INVALID = 1,     /* argument validation failed (the reference returns an error) */
    LTHN_ERR_CUDA = 2,        /* a CUDA runtime call failed */
    LTHN_ERR_UNAVAILABLE = 3, /* no usable device / optional library missing */
    LTHN_ERR_STATE = 4,       /* call not valid in the object's current state */
    LTHN_ERR_DEVICE_WAIT = 5  /* a bounded device-side wait ran out */
};

enum { LTHN_DTYPE_F32 = 0, LTHN_DTYPE_BF16 = 1 };

/* ---- backend discovery: inference.Backend.Available / DeviceInfoProvider ----
 * inference.go:382-400 (Backend), device.go:12-25 (DeviceInfo). */
typedef struct {
    char name[128];          /* e.g. "NVIDIA B200" */
    char architecture[16];   /* "sm_100" */
    uint64_t memory_size;    /* total device memory, bytes */
    uint64_t max_buffer_length;
    uint64_t max_recommended_working_set;
    int32_t sm_count;
    int32_t compute_major, compute_minor;
} lthn_device_info;

const char* lthn_last_error(void);
int32_t lthn_cuda_available(void);              /* 1 when a compute-capability 10.x device is visible; never fails */
int32_t lthn_cuda_device_count(void);
int32_t lthn_cuda_set_device(int32_t device);   /* binds the calling thread (cf. engine/hip/hip_driver_cgo.go:208) */
int32_t lthn_cuda_device_info(int32_t device, lthn_device_info* out);
int32_t lthn_cuda_mem_info(uint64_t* free_bytes, uint64_t* total_bytes); /* engine/memory_reporter.go */
/* Device-side waits (mbarrier phases, peer flags) are bounded: a kernel whose wait runs out sets a
 * bit in a sticky status word and returns, so the context stays usable. The host-buffer entry
 * point, the sessions and the lane sets check that word themselves; after the asynchronous
 * entry points (lthn_affine_qmv, _geglu, _normed, _noalloc, lthn_affine_qmm, lthn_sdpa_decode)
 * call this to learn of it: synchronises `stream`, reads and clears the status words of the
 * current device into *bits (may be NULL) and returns LTHN_ERR_DEVICE_WAIT when any bit was set.
 * Copies four bytes per word to the host; allocates nothing. No counterpart in the reference
 * (its HIP shim reports launch failures through hipGetLastError, engine/hip/hip_driver_cgo.go). */
int32_t lthn_device_status(void* stream, uint32_t* bits);

/* ---- device memory / streams / events: the thin driver wrappers a cgo shim
 * needs (cf. engine/hip/hip_driver_cgo.go:7-670 malloc/free/memcpy/events). ---- */
int32_t lthn_malloc(void** dptr, size_t bytes);
int32_t lthn_free(void* dptr);
int32_t lthn_host_alloc(void** hptr, size_t bytes);  /* pinned host memory */
int32_t lthn_host_free(void* hptr);
int32_t lthn_memcpy_h2d(void* dst, const void* src, size_t bytes, void* stream); /* async when src is pinned */
int32_t lthn_memcpy_d2h(void* dst, const void* src, size_t bytes, void* stream);
int32_t lthn_memcpy_d2d(void* dst, const void* src, size_t bytes, void* stream);
int32_t lthn_memset(void* dst, int32_t value, size_t bytes, void* stream);
int32_t lthn_stream_create(void** stream);
int32_t lthn_stream_destroy(void* stream);
int32_t lthn_stream_sync(void* stream);
int32_t lthn_device_sync(void);
int32_t lthn_event_create(void** event);
int32_t lthn_event_destroy(void* event);
int32_t lthn_event_record(void* event, void* stream);
int32_t lthn_event_elapsed_ms(void* start, void* stop, float* ms); /* synchronises on stop */

/* CUDA-graph capture of a sequence of calls issued on `stream` (the decode loop
 * and the benchmark replay launch-bound kernel chains this way). Call every
 * entry point once un-captured first: first use may allocate scratch memory. */
int32_t lthn_graph_begin(void* stream);
int32_t lthn_graph_end(void* stream, void** graph_exec);
int32_t lthn_graph_launch(void* graph_exec, void* stream);
int32_t lthn_graph_destroy(void* graph_exec);

/* ---- MLX-affine codec on the device ---------------------------------------
 * lthn_affine_quantize: mlxaffine.QuantizeTensor (model/quant/mlxaffine/
 * mlxaffine.go:80-173), bit-exact: f32 [N,K] -> packed/scales/biases.
 * variant 0 = the reference's edge-anchored rule, 1 = literal scale=(max-min)/
 * (2^bits-1), bias=min. bits in {2,4,8}; gs divides K and gs % (32/bits) == 0. */
int32_t lthn_affine_quantize(void* stream, const float* w, int64_t N, int64_t K, int32_t bits, int32_t gs,
                             int32_t variant, uint32_t* packed, uint16_t* scales, uint16_t* biases);
/* lthn_affine_dequantize: mlxaffine.DequantizeTensor (mlxaffine.go:178-208),
 * bit-exact (separately rounded f32 multiply and add). out f32 [N,K]. */
int32_t lthn_affine_dequantize(void* stream, const uint32_t* packed, const uint16_t* scales, const uint16_t* biases,
                               int64_t N, int64_t K, int32_t bits, int32_t gs, float* out);
/* Same dequantisation rounded once more to bf16 (the operand the prefill
 * tensor-core path multiplies with). out bf16 [N,K]. */
int32_t lthn_affine_dequantize_bf16(void* stream, const uint32_t* packed, const uint16_t* scales,
                                    const uint16_t* biases, int64_t N, int64_t K, int32_t bits, int32_t gs,
                                    uint16_t* out);
/* Deterministic synthetic tensors (no counterpart in the reference, which
 * benchmarks downloaded checkpoints): element i of stream `seed` is
 * sigma * IrwinHall8(hash(seed,i)), identical on CPU (oracle) and GPU. */
int32_t lthn_synth_normal_fill(void* stream, uint64_t seed, uint64_t first, int64_t n, float sigma, float* out);
/* Fused generate+quantize of a synthetic [N,K] weight (element index r*K+c). */
int32_t lthn_synth_affine_weight(void* stream, uint64_t seed, float sigma, int64_t N, int64_t K, int32_t bits,
                                 int32_t gs, int32_t variant, uint32_t* packed, uint16_t* scales, uint16_t* biases);

/* ---- affine_qmv: decode-time quantized matvec, M activation rows ------------
 * y[M,N] = x[M,K] * dequant(W[N,K])^T with fp32 accumulation.
 * Replaces: Metal affine_qmv dispatch (engine/metal/qmv.go:282-505,
 * dispatch_sink.go:525-570), M-row lthn_qmv_rows (engine/metal/kernels/quant/
 * lthn_qmv_rows.metal:44-140) and HIP rocm_mlx_q4_projection(_batch)
 * (engine/hip/kernels/quant/affine_projection.hipinc:3-266). All pointers are
 * device pointers. x_dtype/y_dtype: LTHN_DTYPE_*. M in [1,32].
 * bits=4, gs=64 runs the tensor-core streaming kernels; bits=8, gs=64 with one or two
 * rows (N a multiple of 16, 16-byte aligned x and packed) runs the 8-bit form of the
 * integer tensor-core kernel, the code bytes going into the MMA as they are; every other
 * bits in {2,4,8} with gs in {32,64,128} is served by a general kernel. M==0, N==0 or
 * K==0 is a successful no-op (quant_reference_test.go:66-74). */
int32_t lthn_affine_qmv(void* stream, const void* x, int32_t x_dtype, int32_t M, const uint32_t* packed,
                        const uint16_t* scales, const uint16_t* biases, int64_t N, int64_t K, int32_t gs,
                        int32_t bits, void* y, int32_t y_dtype);

/* Allocation-free form of lthn_affine_qmv for f32 activations (4 bit, group 64, f32 out).
 * It has no counterpart in the reference. For hosts that may not allocate device memory
 * while serving (a fixed start-up memory budget, code running where the CUDA allocator
 * must not be entered, launch-only sandboxes): the bf16 activation columns that
 * lthn_affine_qmv stages in a growing arena live here in a fixed 512 KiB array inside the
 * library image (held by every GPU that loads it until exit), so the call performs no
 * cudaMalloc / cudaFree. Limit: 256 + M*s*K*2 <= 524288 bytes with s = 3 for M <= 2 and
 * s = 2 above (e.g. M=1: K <= 87296; M=8: K <= 16320; M=32: K <= 4032); larger sizes are
 * rejected with LTHN_ERR_INVALID. The first call on a device resolves the array's device
 * address (cudaGetSymbolAddress) and should therefore come before any stream capture.
 * All calls on a device share the one array: calls whose kernels can overlap on the GPU
 * (different streams without ordering) race; order them. The array's first word is a sticky
 * status word (a bounded wait that ran out inside the kernel sets it; y is then not valid):
 * lthn_device_status reads and clears it, also without allocating. */
int32_t lthn_affine_qmv_noalloc(void* stream, const float* x, int32_t M, const uint32_t* packed,
                                const uint16_t* scales, const uint16_t* biases, int64_t N, int64_t K, float* y);

/* affine_qmv for 1 or 2 rows with the decoder block's residual RMSNorm pair as its prologue:
 *     h_new = h_in + rmsnorm(a; w_post)        (a == NULL: h_new = h_in, h_out unused)
 *     y     = dequant(W) * rmsnorm(h_new; w_next)
 * and h_new stored to h_out (must not alias h_in). Same arithmetic as lthn_rmsnorm_residual
 * followed by lthn_affine_qmv (hip_gemma4_q4_oracle_test.go:925-951 norms, the HIP affine
 * projection for the product) in one launch - the role of the reference's fused RMSNorm->qmv
 * kernel (engine/metal/kernels/quant/lthn_rms_qmv.metal:23-146), with the residual add included; up_* non-NULL adds the GeGLU epilogue of
 * lthn_affine_qmv_geglu. 4-bit, group 64, N a multiple of 16, f32 vectors 8-byte aligned.
 * Returns LTHN_ERR_INVALID for shapes the batch-1/2 kernel does not serve. The fusion itself
 * has no counterpart in the reference (it runs these steps as separate kernels). */
int32_t lthn_affine_qmv_normed(void* stream, const float* a, const float* h_in, float* h_out, const float* w_post,
                               const float* w_next, float eps, int32_t M, const uint32_t* packed, const uint16_t* scales,
                               const uint16_t* biases, const uint32_t* up_packed, const uint16_t* up_scales,
                               const uint16_t* up_biases, int64_t N, int64_t K, void* y, int32_t y_dtype);

/* The same with the weights' code width given: bits = 4 is lthn_affine_qmv_normed; bits = 8 (group 64,
 * one code per byte - the MLP projections of a mixed-precision pack) runs the same prologue in front of
 * the 8-bit form of the kernel. No counterpart in the reference. */
int32_t lthn_affine_qmv_normed_bits(void* stream, const float* a, const float* h_in, float* h_out, const float* w_post,
                                    const float* w_next, float eps, int32_t M, const uint32_t* packed, const uint16_t* scales,
                                    const uint16_t* biases, const uint32_t* up_packed, const uint16_t* up_scales,
                                    const uint16_t* up_biases, int64_t N, int64_t K, int32_t bits, void* y, int32_t y_dtype);

/* Fused GeGLU pair: y[M,N] = gelu_tanh(x * dequant(Wgate)^T) * (x * dequant(Wup)^T),
 * both weights [N,K], 4 bit, group 64; gate and up rows are streamed together so
 * the activation is read once and the intermediate never reaches memory.
 * Replaces rocm_mlx_q4_gelu_tanh_multiply (engine/hip/kernels/quant/
 * affine_gelu_tanh.hipinc:3-180); gelu as hipGemma4Q4HostGELU
 * (engine/hip/hip_gemma4_q4_layer.go:3582-3597). */
int32_t lthn_affine_qmv_geglu(void* stream, const void* x, int32_t x_dtype, int32_t M, const uint32_t* gate_packed,
                              const uint16_t* gate_scales, const uint16_t* gate_biases, const uint32_t* up_packed,
                              const uint16_t* up_scales, const uint16_t* up_biases, int64_t N, int64_t K, void* y,
                              int32_t y_dtype);
/* The same with the code width given: bits = 4 as above; bits = 8 (group 64, one or two rows) for the
 * gate and up projections of a mixed-precision pack (per-module overrides, model/quant_config.go:39-88). */
int32_t lthn_affine_qmv_geglu_bits(void* stream, const void* x, int32_t x_dtype, int32_t M, const uint32_t* gate_packed,
                                   const uint16_t* gate_scales, const uint16_t* gate_biases, const uint32_t* up_packed,
                                   const uint16_t* up_scales, const uint16_t* up_biases, int64_t N, int64_t K, int32_t bits,
                                   void* y, int32_t y_dtype);

/* ---- affine_qmm: prefill-time quantized matmul on the tensor cores --------------
 * y[M,N] (bf16) = x[M,K] (bf16) * dequant(W[N,K])^T, fp32 accumulation in TMEM.
 * Replaces the Metal engine's affine_qmm_t dispatch (engine/metal/
 * quant_seam_backend.go:84-110, attention.go:731-749) and HIP's
 * rocm_mlx_q4_projection_batch* (engine/hip/kernels/quant/
 * affine_projection_tuned.hipinc:166-559). Weights are dequantised to bf16
 * (one rounding of scale*q+bias) tile by tile in shared memory and multiplied with
 * tcgen05.mma. bits=4 or 8, gs=64, M>32 take the tensor-core kernel (8-bit codes, one per
 * byte, are the MLP projections of mixed-precision packs); other widths and small M are
 * served by the decode kernels. x, y device pointers, 16-byte aligned. */
int32_t lthn_affine_qmm(void* stream, const uint16_t* x, int32_t M, const uint32_t* packed, const uint16_t* scales,
                        const uint16_t* biases, int64_t N, int64_t K, int32_t gs, int32_t bits, uint16_t* y);

/* Prefill GeGLU pair: y[M,N] (bf16) = gelu_tanh(x Wgate^T) * (x Wup^T), both weights [N,K], 4 bit,
 * group 64. One tensor-core pass: a CTA's weight tile holds rows of both matrices, and the
 * epilogue multiplies the two f32 accumulators before the single bf16 rounding, so the
 * intermediate never reaches memory. Replaces rocm_mlx_q4_gelu_tanh_multiply's batched use in
 * prefill (engine/hip/kernels/quant/affine_gelu_tanh.hipinc:3-180). Any M >= 1. */
int32_t lthn_affine_qmm_geglu(void* stream, const uint16_t* x, int32_t M, const uint32_t* gate_packed,
                              const uint16_t* gate_scales, const uint16_t* gate_biases, const uint32_t* up_packed,
                              const uint16_t* up_scales, const uint16_t* up_biases, int64_t N, int64_t K, uint16_t* y);
/* The same with the code width given: bits = 4 as above, bits = 8 for a pair kept at 8 bits (group 64). */
int32_t lthn_affine_qmm_geglu_bits(void* stream, const uint16_t* x, int32_t M, const uint32_t* gate_packed,
                                   const uint16_t* gate_scales, const uint16_t* gate_biases, const uint32_t* up_packed,
                                   const uint16_t* up_scales, const uint16_t* up_biases, int64_t N, int64_t K, int32_t bits,
                                   uint16_t* y);

/* model.QuantMatVec.MatVec (model/quant.go:35-38): bf16 LE bytes in HOST memory
 * in, bf16 LE bytes out; lengths are validated like the reference
 * (enginetest/quant_reference.go:79-104). Copies in, launches, copies out,
 * synchronises. This is what `model.RegisterBackendQuant("cuda", q)` binds. */
int32_t lthn_affine_qmv_host(const void* x, size_t x_len, const void* packed, size_t packed_len,
                             const void* scales, size_t scales_len, const void* biases, size_t biases_len,
                             int64_t out_dim, int64_t in_dim, int32_t gs, int32_t bits, void* y, size_t y_len);

/* ---- fused decoder-step kernels ----------------------------------------------
 * For callers that drive the layer loop themselves; the engine below uses the same
 * kernels. All pointers are device pointers, activations f32.
 *
 * lthn_rmsnorm: hipReferenceRMSNorm (engine/hip/hip_transformer_reference.go:171-194),
 * rocm_rms_norm (engine/hip/kernels/norms/rms_norm.hipinc:28). out[r,:] = x/rms*w. */
int32_t lthn_rmsnorm(void* stream, const float* x, const float* w, float* out, int32_t rows, int32_t width, float eps);
/* h += norm(a, w_post); out = norm(h, w_next): the fused post-norm + residual + next
 * pre-norm of rocm_rms_norm_residual_add_norm (rms_norm.hipinc) / lthn_rmsnorm_residual_bf16. */
int32_t lthn_rmsnorm_residual(void* stream, const float* a, float* h, const float* w_post, const float* w_next,
                              float* out, int32_t rows, int32_t width, float eps);
/* lthn_rmsnorm_rope: per-head RMSNorm then NeoX RoPE over the first rotary_dim dims
 * (pairs (i, i+head_dim/2)), one position per row; head_dim <= 512.
 * Replaces lthn_qknorm_rope_bf16(_rows) (engine/metal/kernels/norms/
 * lthn_qknorm_rope_bf16.metal:28-206) and rocm_rms_norm_rope_heads (rms_norm.hipinc:
 * 306-377); CPU refs hip_transformer_reference.go:171-194,242-289. x/out [rows,
 * heads*head_dim] f32. bf16_seams=1 reproduces the Metal kernel's bf16 rounding points
 * (bf16(w*bf16(x*inv)), bf16 output values). */
int32_t lthn_rmsnorm_rope(void* stream, const float* x, const float* w, const int32_t* positions, float* out,
                          int32_t rows, int32_t heads, int32_t head_dim, int32_t rotary_dim, float eps, float rope_base,
                          int32_t bf16_seams);
/* lthn_sdpa_decode: softmax(q K^T scale) V for `rows` single-token queries over the
 * seq-major bf16 KV cache (cache row p of lane l at l*lane_stride + p*kv_heads*head_dim;
 * engine/metal/decode_step.go:20-26), keys 0..row_pos[r] inclusive, GQA head map
 * kv = q_head / (q_heads/kv_heads). Split-KV with a log-sum-exp merge; partials live in a
 * library-owned scratch arena. Replaces sdpa_vector(_2pass) routing (engine/metal/sdpa.go:
 * 520-545) and rocm_attention_heads(_chunked) (engine/hip/kernels/attention/); CPU ref
 * hipReferenceSingleHeadAttentionWithScale (hip_transformer_reference.go:295-330).
 * q/out [rows, q_heads*head_dim] f32; scale<=0 means 1/sqrt(head_dim); max_ctx bounds
 * row_pos+1 and sizes the grid. head_dim in {64,128,256,512}. */
int32_t lthn_sdpa_decode(void* stream, const float* q, const uint16_t* kcache, const uint16_t* vcache,
                         const int32_t* row_pos, const int32_t* row_lane, float* out, int32_t rows, int32_t q_heads,
                         int32_t kv_heads, int32_t head_dim, int64_t lane_stride, float scale, int32_t max_ctx);
/* lthn_prefill_attention: causal attention for `rows` consecutive prompt positions pos0 ..
 * pos0+rows-1 of one cache lane, whose K and V rows (the chunk's own included) are already in the
 * cache: row r attends keys 0 .. pos0+r. Same cache layout and head map as lthn_sdpa_decode
 * (kcache/vcache point at the lane's first row; row stride kv_heads*head_dim). Tensor-core
 * kernel with the bf16 contract of the reference's Metal prefill: q and the softmax weights are
 * rounded to bf16 for the two products, scores and output accumulate in f32; out is bf16
 * [rows, q_heads*head_dim], ready to be the next affine_qmm's x. Stands where the reference
 * prefills with its batched chunked attention (engine/hip/kernels/attention/chunked.hipinc) /
 * MLX's sdpa over the chunk; CPU ref hipReferenceSingleHeadAttentionWithScale
 * (hip_transformer_reference.go:295-330). head_dim in {64,128,256}; scale<=0 means 1/sqrt(head_dim). */
int32_t lthn_prefill_attention(void* stream, const float* q, const uint16_t* kcache, const uint16_t* vcache, uint16_t* out,
                               int32_t rows, int32_t pos0, int32_t q_heads, int32_t kv_heads, int32_t head_dim, float scale);
/* Greedy pick per row: strict '>', lowest index wins ties (model.Greedy, model/sample.go:
 * 29-50; hipReferenceGreedySample). logits [rows, vocab] f32. */
int32_t lthn_argmax(void* stream, const float* logits, int32_t rows, int32_t vocab, int32_t* out_idx);

/* ---- the engine: engine.TokenModel / engine.Session / inference.LaneSet ----------
 * A Gemma-style decoder (gemma3 block: four norms, per-head Q/K norm, full NeoX
 * rotary, GeGLU, tied embedding/lm_head; model/arch/google/gemma3/gemma3.go:141-161)
 * over resident MLX-affine 4-bit weights and a seq-major bf16 KV cache. */
typedef struct {
    int32_t layers, hidden, q_heads, kv_heads, head_dim, ffn, vocab;
    int32_t group_size, bits;   /* 64, 4 */
    int32_t max_len;            /* KV positions per lane (LoadConfig.ContextLen, options.go:281-288) */
    int32_t max_lanes;          /* resident KV lanes: sessions + lane-set lanes (LoadConfig.ParallelSlots) */
    float eps;                  /* 0 -> 1e-6 */
    float rope_base;            /* 0 -> 10000 */
    float attn_scale;           /* 0 -> 1/sqrt(head_dim) (model.Arch.AttnScale) */
    float embed_scale;          /* 0 -> bf16(sqrt(hidden)) (model.Arch.EmbedScale) */
    int32_t tp_rank, tp_size;   /* tensor-parallel rank / degree (tp_size 0 or 1: single GPU) */
    /* gemma3 sliding/global attention (model/arch/google/gemma3/gemma3.go:111-158): with sliding_window > 0,
     * block i attends only the last sliding_window keys (the current one included) unless
     * (i+1) % sliding_pattern == 0 (pattern 0 -> 6), and rotates q/k with rope_local_base (0 -> 10000)
     * instead of rope_base. The cache keeps every row (no ring): what the reference's ring of
     * sliding_window rows computes (engine/metal/decode_step.go:298-316), without its memory saving. */
    int32_t sliding_window, sliding_pattern;
    float rope_local_base;
} lthn_model_config;

enum { LTHN_ROLE_Q = 0, LTHN_ROLE_K, LTHN_ROLE_V, LTHN_ROLE_O, LTHN_ROLE_GATE, LTHN_ROLE_UP, LTHN_ROLE_DOWN };
enum { LTHN_NORM_INPUT = 0, LTHN_NORM_POST_ATTN, LTHN_NORM_PRE_FF, LTHN_NORM_POST_FF, LTHN_NORM_Q, LTHN_NORM_K };

/* Backend.LoadModel's device half (inference.go:394; engine/hip/inference_model.go:402):
 * create, upload every tensor of model.LoadedModel (model/loaded.go:157-175), finalize.
 * Uploads take HOST pointers to the full (unsharded) MLX-affine tensors - exactly the
 * byte slices of model.Linear (model/linear.go:21-29) - and copy what this rank owns;
 * nothing is retained, so the safetensors mmap may be closed afterwards. layer < 0 names
 * the token embedding (tied lm_head) / the final norm. Norm weights are the effective
 * weights (the gemma "(1+w)" fold of model/norm_bias.go:22-49 applied by the loader). */
int32_t lthn_model_create(const lthn_model_config* cfg, void** model);
int32_t lthn_model_upload_linear(void* model, int32_t layer, int32_t role, const void* packed, const void* scales,
                                 const void* biases, int64_t N, int64_t K);
/* The same for a linear whose quantization override names its own code width (the mixed-precision
 * QAT packs of model/quant_config.go:39-88 keep the MLP projections at 8 bits). bits = 4 is
 * lthn_model_upload_linear; bits = 8 (group 64) is accepted for LTHN_ROLE_GATE / UP / DOWN on one
 * GPU: packed holds N*K bytes, one code per byte. Decode steps of one and two rows run the 8-bit form
 * of the integer tensor-core matvec, prompts and steps of 3..32 rows the 8-bit form of the prefill GEMM
 * (bf16-rounded activations; LTHN_CUDA_BATCH_F32=1 keeps such steps on an f32-grade kernel); a block whose gate and
 * up projections differ in width runs them as separate matvecs followed by a GeGLU kernel, and a model
 * with such a block keeps its norms unfused and its prompts on the batched matvec path. */
int32_t lthn_model_upload_linear_bits(void* model, int32_t layer, int32_t role, const void* packed, const void* scales,
                                      const void* biases, int64_t N, int64_t K, int32_t bits);
int32_t lthn_model_upload_norm(void* model, int32_t layer, int32_t role, const float* w, int64_t n);
/* Synthetic weights (benchmarks, tests): tensor (layer, role) is the seeded synthetic
 * [N,K] tensor of stream seed*1000003 + (layer+1)*16 + role quantised with the
 * reference rule; norms are 1. No counterpart in the reference. */
int32_t lthn_model_synthesize(void* model, uint64_t seed, float sigma);
int32_t lthn_model_finalize(void* model);
int32_t lthn_model_weight_bytes(void* model, uint64_t* bytes);
/* How a finalized model combines the partial sums of its row-parallel projections:
 * 0 single device, 1 NCCL all-reduce, 2 peer-memory exchange fused into the residual RMSNorm
 * (CUDA IPC mappings of every rank's buffer; chosen when every rank could map every peer,
 * LTHN_CUDA_TP_NCCL=1 forces mode 1). No counterpart in the reference. */
int32_t lthn_model_tp_exchange(void* model, int32_t* mode);
/* Whether decode steps replay a captured CUDA graph: 0 not captured yet, 1 graph, 2 capture was
 * not possible (kernel-by-kernel launches; LTHN_CUDA_NO_GRAPH=1 forces this). No counterpart in the reference. */
int32_t lthn_model_graph_state(void* model, int32_t* state);
/* How a finalized model runs a one-row decode step: 0 a chain of per-op kernels (the default), 1 one
 * cooperative kernel for all decoder blocks (opt-in with LTHN_CUDA_PERSIST=1 at finalize; one GPU,
 * two query heads per kv head, head_dim 64 / 128 / 256, hidden <= 5632). Steps of more rows,
 * prompts and tensor-parallel models always take the chain. No counterpart in the reference. */
int32_t lthn_model_decode_kernel(void* model, int32_t* mode);
int32_t lthn_model_destroy(void* model);   /* TokenModel.Close (engine/model.go:30) */

/* model.Load (model/load.go:19-108) for a gemma3-style MLX-affine checkpoint directory: reads
 * config.json (text fields at top level or under "text_config"; "quantization" block with
 * group_size / bits and per-module overrides, model/quant_config.go:39-88) and the safetensors
 * directory (model.safetensors, or the shards model.safetensors.index.json names; tensor names of
 * model/assemble.go:56-75, an optional "language_model." prefix stripped), checks every linear's
 * geometry against the quantization block as affineGeometry does (model/linear.go:91-102), widens
 * F16 scales/biases/norms to bf16 (model/safetensors/widen.go), applies the gemma (1+w) norm fold
 * in the tensor's dtype (model/norm_bias.go:22-49), uploads this rank's shard of every tensor and
 * finalizes. The files are mapped read-only for the duration of the call. Linears are 4-bit /
 * group 64; an 8-bit / group-64 per-module override is taken on the MLP projections of a one-GPU
 * model (lthn_model_upload_linear_bits); anything else is rejected with the tensor named. A
 * checkpoint with sliding_window runs gemma3's layer pattern (sliding blocks with
 * rope_local_base_freq, every sliding_window_pattern-th block global); uniform_attention = 1 runs
 * every block with full attention and the checkpoint's rope_theta instead. */
typedef struct {
    int32_t max_len;            /* KV positions per lane; 0 -> min(max_position_embeddings, 4096) */
    int32_t max_lanes;          /* 0 -> 1 */
    int32_t tp_rank, tp_size;   /* tensor-parallel shard to keep (tp_size 0 or 1: everything) */
    void* comm;                 /* communicator from lthn_tp_init when tp_size > 1 */
    int32_t uniform_attention;
} lthn_load_options;
int32_t lthn_model_load_dir(const char* dir, const lthn_load_options* opts, void** model);
/* The host half of the same: parses config.json and the safetensors directories and writes a
 * one-line JSON summary (dimensions, quantization, tensor and shard counts) into json_out. Needs
 * no device. */
int32_t lthn_checkpoint_inspect(const char* dir, char* json_out, size_t json_len);

/* Tensor parallelism over NCCL (the reference is single-device; new functionality).
 * Rank 0 makes the id, the host distributes its 128 bytes, every rank joins. */
int32_t lthn_tp_unique_id(void* out128);
int32_t lthn_tp_init(int32_t rank, int32_t world, const void* id128, void** comm);
int32_t lthn_tp_destroy(void* comm);
int32_t lthn_model_set_comm(void* model, void* comm);

/* Prompts of more than 32 tokens are prefilled in chunks of up to 2048 rows (the reference's
 * chunks are 512, decode/generate/generate.go:147-150; a B200 wants more tiles in flight) through
 * lthn_affine_qmm and lthn_prefill_attention, the route the reference takes for
 * M > 1 (engine/metal/quant_seam_backend.go:37-68), with that engine's bf16 contract: activations
 * entering a projection and the dequantised weights are bf16, everything else f32. Shorter prompts
 * and appended pieces go through the f32 decode kernels, 32 rows per forward, as every prompt
 * does when LTHN_CUDA_PREFILL_F32=1 is set at lthn_model_create (or head_dim is 512).
 *
 * engine.Session (engine/session.go:40-61). One session is driven by one host thread at
 * a time (SessionHandle.mu, engine/session.go:105-117); sessions of one model serialise
 * on the model's stream. */
int32_t lthn_session_open(void* model, void** session);                      /* TokenModel.OpenEngineSession */
int32_t lthn_session_prefill(void* session, const int32_t* ids, int32_t n); /* PrefillTokens: replaces state */
int32_t lthn_session_append(void* session, const int32_t* ids, int32_t n);  /* AppendTokens */
int32_t lthn_session_pos(void* session);                                     /* Pos */
/* GenerateFromCacheEach: up to max_new greedy tokens into out_ids; eos_id < 0 leaves the
 * stop decision to the caller (the Go side calls this in small chunks so `yield` can
 * stop it). The last produced token stays pending and is fed by the next call. */
int32_t lthn_session_decode_greedy(void* session, int32_t max_new, int32_t eos_id, int32_t* out_ids, int32_t* n_out);
/* Logits after the last fed token, for GenerateSampledFromCacheEach's host-side sampler. The
 * buffer behind it belongs to the model: LTHN_ERR_STATE when another session or lane set of the
 * model has run a forward since this session's last one. */
int32_t lthn_session_logits(void* session, float* logits_host, int64_t n);
/* CaptureKVWithOptions / RestoreFromKV payloads (kv/snapshot.go:98-143): one layer's keys
 * (which=0) or values (which=1) as bf16 [pos, kv_heads_local*head_dim]. */
int32_t lthn_session_kv_export(void* session, int32_t layer, int32_t which, void* out_host, size_t out_bytes);
int32_t lthn_session_kv_import(void* session, int32_t layer, int32_t which, const void* in_host, int32_t tokens);
int32_t lthn_session_set_state(void* session, int32_t pos, int32_t pending_token);
/* kv.Snapshot by token ranges (kv/snapshot.go:98-143; Session.RangeKVBlocks and CaptureOptions.BlockStartToken,
 * engine/session.go:53-58): rows [token0, token0+ntokens) of a layer's K (which = 0) or V (1), ntokens x
 * (local kv heads * head_dim) bf16 values. Export reads below the session's position, import may write
 * anywhere below the context length (follow it with lthn_session_set_state). */
int32_t lthn_session_kv_export_range(void* session, int32_t layer, int32_t which, int32_t token0, int32_t ntokens, void* out_host,
                                     size_t out_bytes);
int32_t lthn_session_kv_import_range(void* session, int32_t layer, int32_t which, int32_t token0, const void* in_host, int32_t ntokens);
/* The same rows with the kv heads of every tensor-parallel rank, in model order (ntokens x kv_heads *
 * head_dim): every rank calls it with the same arguments (one NCCL all-gather) and gets the full rows. */
int32_t lthn_session_kv_gather_range(void* session, int32_t layer, int32_t which, int32_t token0, int32_t ntokens, void* out_host,
                                     size_t out_bytes);
/* Session.Fork / Session.Reset (engine/enginetest/session.go:72-105): a copy of the session on a KV lane of
 * its own (the model needs a free lane); forget the sequence. */
int32_t lthn_session_fork(void* session, void** fork);
int32_t lthn_session_reset(void* session);
/* engine.DecodePhaseTracer (engine/session.go:86-98) with inference.DecodePhaseBudget
 * (inference.go:218-268): lthn_session_trace_begin turns per-token phase timing on for the one-row
 * decode steps that follow on this session's model; lthn_session_trace_end turns it off and returns
 * the averages over the traced steps. While a trace is on, steps run kernel by kernel (no CUDA-graph
 * replay) with CUDA events between the phases, so total_per_token_us is the traced wall time, not the
 * untraced speed. Without traced steps the budget is all zeros. A single-flight diagnostic. */
typedef struct {
    int32_t tokens;               /* decode steps the aggregate is averaged over */
    double total_per_token_us;    /* wall time from begin to end, per step */
    double gpu_per_token_us;      /* device time between the first and the last event of a step */
    int32_t n_phases;
    struct {
        char name[48];
        double per_token_us;
        int32_t gpu;              /* 1: device time */
    } phases[8];
} lthn_decode_phase_budget;
int32_t lthn_session_trace_begin(void* session);
int32_t lthn_session_trace_end(void* session, lthn_decode_phase_budget* budget);
int32_t lthn_session_close(void* session);

/* ---- sampling: model.Sampler / model.SampleParams (model/sample.go:52-400) ------------------
 * The reference's sampler draws from bf16 logits with a splitmix64 stream that advances once per
 * stochastic token: temperature (<= 0: greedy), top-k, top-p, min-p, suppressed tokens, and a
 * repeat penalty over the tokens generated so far (sample.go:449-508; > 1 engages it).
 * lthn_sampler_* is that sampler on host buffers, operation for operation, so a given seed gives
 * the reference's tokens. */
typedef struct {
    float temperature;
    int32_t top_k;
    float top_p, min_p;
    float repeat_penalty;
    int32_t min_tokens_before_stop;   /* stop tokens are suppressed until this many tokens were generated */
    const int32_t* suppress;          /* SuppressTokens */
    int32_t n_suppress;
} lthn_sample_params;
int32_t lthn_sampler_create(uint64_t seed, void** sampler);           /* model.NewSampler */
int32_t lthn_sampler_destroy(void* sampler);
float lthn_sampler_draw(void* sampler);                               /* Sampler.Draw */
/* Sampler.Sample: logits = vocab bf16 values in host memory. */
int32_t lthn_sampler_sample(void* sampler, const uint16_t* logits_bf16, int32_t vocab, const lthn_sample_params* params, int32_t* token);
/* Sampler.SampleCandidates: n candidate values with the token ids they belong to. */
int32_t lthn_sampler_sample_candidates(void* sampler, const uint16_t* logits_bf16, const int32_t* ids, int32_t n,
                                       const lthn_sample_params* params, int32_t* token);
/* Device half: the k best entries of each f32 logit row after rounding to bf16, by (value
 * descending, index ascending) - the order of selectTopKDesc (sample.go:339-366) - as k ids and
 * bf16 values per row at out_ids / out_bf16 + row*256, unordered within the k. k <= min(256, vocab).
 * scratch_bf16: rows*vocab bf16 values of device memory. Replaces the reference's device top-k
 * (engine/hip/kernels/sampling/topk.hipinc). */
int32_t lthn_topk_candidates(void* stream, const float* logits, int32_t rows, int32_t vocab, int32_t k, uint16_t* scratch_bf16,
                             int32_t* out_ids, uint16_t* out_bf16);
/* GenerateSampledFromCacheEach (engine/session.go:51, loop of model/token.go:263-305): up to max_new
 * tokens drawn with `sampler` from the session's logits; the repeat penalty sees the tokens of this
 * call; a token in `stop` ends the call after it is emitted (and is suppressed while fewer than
 * min_tokens_before_stop tokens were generated). With 1 < top_k <= 256 only the top-k window leaves
 * the device each step; other settings read the bf16 row back. The last token is not fed. */
int32_t lthn_session_decode_sampled(void* session, void* sampler, const lthn_sample_params* params, int32_t max_new,
                                    const int32_t* stop, int32_t n_stop, int32_t* out_ids, int32_t* n_out);

/* inference.LaneSet (batch_step.go:97-119) behind engine.LaneSetOpener
 * (engine/batch_step.go:21-23). Single host thread per set. */
int32_t lthn_laneset_open(void* model, int32_t max_lanes, void** set);
int32_t lthn_laneset_prepare(void* set, const int32_t* ids, int32_t n, int32_t max_new, const int32_t* stop,
                             int32_t n_stop, int32_t* lane_handle);           /* lane ids start at 1 */
/* LaneSpec.Sampler / SampleSeed (batch_step.go:55-71): a lane with its own sampler state, token-identical
 * to lthn_session_decode_sampled at the same seed and parameters. */
int32_t lthn_laneset_prepare_sampled(void* set, const int32_t* ids, int32_t n, int32_t max_new, const int32_t* stop,
                                     int32_t n_stop, const lthn_sample_params* params, uint64_t seed, int32_t* lane_handle);
int32_t lthn_laneset_step(void* set, int32_t* lane_handles, int32_t* tokens, int32_t* flags, int32_t* n);
int32_t lthn_laneset_retire(void* set, int32_t lane_handle);
int32_t lthn_laneset_active(void* set);
uint64_t lthn_laneset_batch_forward_count(void* set);
int32_t lthn_laneset_close(void* set);

#ifdef __cplusplus
}
#endif
#endif /* LTHN_CUDA_H */
