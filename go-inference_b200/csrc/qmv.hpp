// qmv.hpp — internal interface between the affine_qmv entry points and its kernels.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace lthn {

// Optional prologue of the batch-1/2 kernel: the activations are not read from x but computed
// as the residual RMSNorm pair of the decoder block,
//     h_new = h_in + norm(a; w_post)      (skipped when a is NULL: h_new = h_in)
//     x     = norm(h_new; w_next)
// with the arithmetic of the stand-alone norm kernel (f64 sum of squares, IEEE divide). Every
// CTA computes the whole vector (it needs the sums), CTA 0 also stores h_new to h_out, which
// must not alias h_in. Removes one kernel launch per norm from the decode chain.
//
// Tensor parallel form (wait != NULL): a is the sum of na partial vectors a[r*a_stride + ...], one
// per rank, that the ranks' projection kernels pushed into this GPU's memory. CTA 0 signals the
// exchange's sequence number to every peer, every CTA waits (bounded polling) until all peers have
// signalled, then the partials are added in rank order. Same protocol and counters as the
// stand-alone tensor-parallel norm kernel.
struct PeerWait {
    uint32_t* flag_out[8];    // rank r's flag line as mapped here; element [rank] is this rank's
    const uint32_t* flag_in;  // this rank's flag line
    uint32_t* ctr;            // [0] sequence number of the last finished exchange, [1] CTA arrivals
    int t, rank;
};
struct NormFuse {
    const float* a;
    const float* h_in;
    float* h_out;
    const float* w_post;
    const float* w_next;
    float eps;
    int na = 1;
    int64_t a_stride = 0;
    const PeerWait* wait = nullptr;  // in device memory
    double inv_width = 0.0;          // 1 / vector width, set by the launcher
};

// One decode matvec: y[M,N] = x[M,K] * dequant(W)^T, optionally fused with a second
// weight set as gelu_tanh(W x) * (W2 x). 4-bit codes, group 64.
struct QmvCall {
    const uint32_t* wq; const uint16_t* scales; const uint16_t* biases;
    const uint32_t* wq2; const uint16_t* scales2; const uint16_t* biases2;  // NULL unless fused GeGLU
    const void* x; int x_dtype;
    void* y; int y_dtype;
    int64_t N, K;
    int M;
    // optional: the same activations already split into bf16 columns ([M*x_split, K], column
    // m*x_split+j) by the kernel that produced x; used when the tensor-core kernel is chosen
    const uint16_t* x_cols = nullptr;
    int x_split = 0;
    const NormFuse* norm = nullptr;  // x is ignored when set (integer tensor-core kernel only)
    // optional: the caller sums K-slice partials itself. When parts is set the kernel may leave
    // *nparts (1..8) partial results [nparts][M][N] f32 there instead of y; without it a sliced
    // plan is followed by a small summing kernel.
    float* parts = nullptr;
    int* nparts = nullptr;
    // optional (integer tensor-core kernel, f32 output): store the result to npush buffers instead
    // of y - a tensor-parallel rank pushing its partial sums into every peer's memory
    float* const* push = nullptr;  // array of npush pointers, in device memory
    int npush = 0;
    int bits = 4;  // 8: the integer tensor-core kernel's 8-bit form (plain matvec, M <= 2)
};

// true when a call of this shape can carry a fused norm prologue
bool qmv_can_fuse_norm(int64_t N, int64_t K, int M, bool geglu, int bits = 4);

// bf16 columns a tensor-core matvec over f32 activations wants per activation row
int32_t qmv_split_for(int M, int x_dtype);

struct Dp4aPlan { int J, R, T_row, S, threads, cons_threads, nblocks, part_bytes; size_t smem; };

// dp4a kernel (1-2 activation rows). dp4a_plan returns false when the shape is not served.
bool dp4a_plan(int64_t N, int64_t K, int M, int fuse, int force_r, int force_s, Dp4aPlan* p);
int32_t dp4a_launch(cudaStream_t st, const QmvCall& c, const Dp4aPlan& p);

// Integer tensor-core kernel (1-2 activation rows, N a multiple of 16).
struct I8Plan { int J, W, RT, stg, RS, nblocks, threads, bs_off, stage_off, ks, Gs, fuse; size_t smem; };
extern __attribute__((visibility("hidden"))) int g_i8_stg;
// max_slices: 1 = whole rows only; > 1 lets the plan cut K into up to that many slices (partial sums)
bool i8_plan(int64_t N, int64_t K, int M, int fuse, int force_ks, int force_w, I8Plan* p, int max_slices = 1,
             bool has_norm = false);
bool i8_plan_b8(int64_t N, int64_t K, int M, I8Plan* p, int force_ks = 0, int force_w = 0, int fuse = 0, bool has_norm = false);
int32_t i8_launch(cudaStream_t st, const QmvCall& c, const I8Plan& p);

// y[i] = sum over s < ks of part[s*n + i]
int32_t launch_sum_parts(cudaStream_t st, const float* part, int ks, int64_t n, void* y, int y_dtype);

// One prefill matmul on the tensor cores: y[M,N] = x[M,K] (bf16) * dequant(W)^T, or with a second
// weight set gelu_tanh(x Wgate^T) * (x Wup^T). y is bf16, or f32 when y_f32.
struct QmmCall {
    const uint16_t* x; int M;
    const uint32_t* wq; const uint16_t* scales; const uint16_t* biases;
    const uint32_t* wq2; const uint16_t* scales2; const uint16_t* biases2;
    int64_t N, K;
    void* y; int y_f32;
    int bits = 4;  // 8: one code per byte (both sets of a GeGLU pair)
};
int32_t qmm_launch(cudaStream_t st, const QmmCall& c);

// Tensor-core streaming kernel for up to 32 activation rows (qmv_tc.cu): bf16 activations (row
// pitch x_ld elements), weights dequantised to bf16 (the numeric contract of affine_qmm), f32
// accumulation in TMEM.
bool qmv_tc_available(const QmvCall& c);
int32_t qmv_tc_launch(cudaStream_t st, const QmvCall& c, const uint16_t* x_bf16, int64_t x_ld);
// LTHN_CUDA_BATCH_F32=1 keeps every row count on the f32-grade kernels (read at every call)
bool qmv_batch_f32();
// f32 rows -> `split` bf16 columns per row ([M*split, K]; the first is the bf16 rounding of the value)
int32_t split_f32_launch(cudaStream_t s, const float* x, int64_t M, int64_t K, int split, uint16_t* out);

// Dispatcher used by the C entry points and by the decoder engine.
int32_t qmv_dispatch(cudaStream_t st, const QmvCall& c);

}  // namespace lthn
