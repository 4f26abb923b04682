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
 * bits=4, gs=64 runs the tensor-core streaming kernel; bits in {2,4,8} with
 * gs in {32,64,128} is served by a general kernel. M==0, N==0 or K==0 is a
 * successful no-op (quant_reference_test.go:66-74). */
int32_t lthn_affine_qmv(void* stream, const void* x, int32_t x_dtype, int32_t M, const uint32_t* packed,
                        const uint16_t* scales, const uint16_t* biases, int64_t N, int64_t K, int32_t gs,
                        int32_t bits, void* y, int32_t y_dtype);

/* model.QuantMatVec.MatVec (model/quant.go:35-38): bf16 LE bytes in HOST memory
 * in, bf16 LE bytes out; lengths are validated like the reference
 * (enginetest/quant_reference.go:79-104). Copies in, launches, copies out,
 * synchronises. This is what `model.RegisterBackendQuant("cuda", q)` binds. */
int32_t lthn_affine_qmv_host(const void* x, size_t x_len, const void* packed, size_t packed_len,
                             const void* scales, size_t scales_len, const void* biases, size_t biases_len,
                             int64_t out_dim, int64_t in_dim, int32_t gs, int32_t bits, void* y, size_t y_len);

#ifdef __cplusplus
}
#endif
#endif /* LTHN_CUDA_H */
