// codec.cu — MLX-affine quantise / dequantise on the device, bit-exact with the
// reference's CPU code (go/model/quant/mlxaffine/mlxaffine.go:80-241), plus the
// synthetic-tensor generator shared with the CPU oracle.
//
// Both kernels are pure streaming passes (HBM-bound):
//   dequantise: reads 0.5625 B, writes 4 B (f32) or 2 B (bf16) per element
//   quantise:   reads 4 B, writes 0.5625 B per element
// Every IEEE operation the Go code performs is issued with an explicit
// round-to-nearest intrinsic so the compiler cannot contract a*b+c into an FMA.
#include "common.cuh"

namespace lthn {

// ---- synthetic normal (Irwin-Hall over eight hashed 16-bit uniforms) ---------
__host__ __device__ inline uint64_t splitmix64(uint64_t z) {
    z += 0x9e3779b97f4a7c15ull;
    z = (z ^ (z >> 30)) * 0xbf58476d1ce4e5b9ull;
    z = (z ^ (z >> 27)) * 0x94d049bb133111ebull;
    return z ^ (z >> 31);
}
__device__ __forceinline__ float synth_value(uint64_t seed, uint64_t idx, float k) {
    uint64_t a = splitmix64(seed * 0xd1342543de82ef95ull + 2 * idx);
    uint64_t b = splitmix64(seed * 0xd1342543de82ef95ull + 2 * idx + 1);
    int32_t s = 0;
#pragma unroll
    for (int j = 0; j < 4; j++) {
        s += (int32_t)((a >> (16 * j)) & 0xffff);
        s += (int32_t)((b >> (16 * j)) & 0xffff);
    }
    return __fmul_rn((float)(s - 262140), k);
}
static inline float synth_scale(float sigma) { return sigma * (1.0f / 53509.03f); }

__global__ void synth_fill_kernel(uint64_t seed, uint64_t first, int64_t n, float k, float* __restrict__ out) {
    int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (; i < n; i += stride) out[i] = synth_value(seed, first + (uint64_t)i, k);
}

// ---- dequantise -----------------------------------------------------------
// One thread per packed word (32/bits codes). Threads of a warp read consecutive
// words (coalesced 128 B) and write consecutive 32/bits-element runs.
template <int BITS, bool OUT_BF16>
__global__ void dequant_kernel(const uint32_t* __restrict__ packed, const uint16_t* __restrict__ scales,
                               const uint16_t* __restrict__ biases, int64_t N, int64_t K, int gs,
                               void* __restrict__ out) {
    constexpr int EPW = 32 / BITS;
    const int64_t wpr = K / EPW, gpr = K / gs;
    const int64_t total = N * wpr;
    int64_t widx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (; widx < total; widx += stride) {
        const int64_t r = widx / wpr, wc = widx - r * wpr;
        const int64_t j0 = wc * EPW;
        const uint32_t word = __ldg(packed + widx);
        float v[EPW];
#pragma unroll
        for (int p = 0; p < EPW; p++) {
            // a group is a multiple of EPW codes, but gs may be smaller than a run of 8 only for bits<4
            const int64_t g = (j0 + p) / gs;
            const float s = bf16_bits_to_f32(__ldg(scales + r * gpr + g));
            const float b = bf16_bits_to_f32(__ldg(biases + r * gpr + g));
            const uint32_t code = (word >> (p * BITS)) & ((1u << BITS) - 1u);
            v[p] = __fadd_rn(__fmul_rn(s, (float)code), b);  // mlxaffine.go:204
        }
        if (OUT_BF16) {
            uint16_t* o = (uint16_t*)out + r * K + j0;
#pragma unroll
            for (int p = 0; p < EPW; p++) o[p] = f32_to_bf16_bits(v[p]);
        } else {
            float* o = (float*)out + r * K + j0;
#pragma unroll
            for (int p = 0; p < EPW; p++) o[p] = v[p];
        }
    }
}

// ---- quantise ----------------------------------------------------------------
// A group of GS values is handled by GS/8 consecutive lanes, 8 values each
// (two float4 loads per lane, consecutive lanes contiguous -> coalesced). The
// lanes of a group reduce min/max with xor-shuffles, derive (scale,bias) with the
// exact operation sequence of affineGroup (mlxaffine.go:136-161), then each lane
// emits its 8 codes: one u32 word at 4 bits, two at 8 bits, half a word at 2 bits
// (combined with its neighbour by shuffle).
struct MemSource {
    const float* w;
    __device__ __forceinline__ void load8(int64_t idx, float (&v)[8]) const {
        const float4 a = __ldg((const float4*)(w + idx));
        const float4 b = __ldg((const float4*)(w + idx) + 1);
        v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
    }
};
// Element (r,c) of the local [N,Klocal] tensor is element (r+row0, c+col0) of a full
// tensor with Kfull columns, so a tensor-parallel shard draws the same values as the
// unsharded tensor.
struct SynthSource {
    uint64_t seed; float k;
    int64_t Klocal, Kfull, row0, col0;
    __device__ __forceinline__ void load8(int64_t idx, float (&v)[8]) const {
        const int64_t r = idx / Klocal, c = idx - r * Klocal;
        const int64_t g = (r + row0) * Kfull + c + col0;
#pragma unroll
        for (int i = 0; i < 8; i++) v[i] = synth_value(seed, (uint64_t)(g + i), k);
    }
};

__device__ __forceinline__ float round_half_away(float v) { return roundf(v); }  // mlxaffine.go:213

template <int BITS, typename Source>
__global__ void quantize_kernel(Source src, int64_t N, int64_t K, int gs, int variant,
                                uint32_t* __restrict__ packed, uint16_t* __restrict__ scales,
                                uint16_t* __restrict__ biases) {
    const int lanes_per_group = gs >> 3;  // 4, 8 or 16 (gs 32/64/128); power of two
    const int64_t total8 = N * K / 8;
    const int64_t span = (int64_t)gridDim.x * blockDim.x;
    const float nbins = (float)((1 << BITS) - 1);
    // all lanes of a warp iterate together (total8 is a multiple of lanes_per_group and the
    // loop bound is rounded up to a warp) so the shuffles below are always converged
    const int64_t total8_up = (total8 + 31) / 32 * 32;
    for (int64_t t8 = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; t8 < total8_up; t8 += span) {
        const bool live = t8 < total8;
        const int64_t e0 = (live ? t8 : 0) * 8;
        float v[8];
        src.load8(e0, v);
        float wmin = v[0], wmax = v[0];
#pragma unroll
        for (int i = 1; i < 8; i++) { wmin = fminf(wmin, v[i]); wmax = fmaxf(wmax, v[i]); }
        for (int o = 1; o < lanes_per_group; o <<= 1) {
            wmin = fminf(wmin, __shfl_xor_sync(0xffffffffu, wmin, o));
            wmax = fmaxf(wmax, __shfl_xor_sync(0xffffffffu, wmax, o));
        }
        float scale = __fdiv_rn(__fsub_rn(wmax, wmin), nbins);
        if (scale < 1e-7f) scale = 1e-7f;
        float bias;
        if (variant == 1) {
            bias = wmin;
        } else {
            float edge = wmax;
            if (fabsf(wmin) > fabsf(wmax)) edge = wmin; else scale = -scale;
            const float q0 = round_half_away(__fdiv_rn(edge, scale));
            if (q0 == 0.0f) { bias = 0.0f; } else { scale = __fdiv_rn(edge, q0); bias = edge; }
        }
        uint32_t codes[8];
#pragma unroll
        for (int i = 0; i < 8; i++) {
            float q = round_half_away(__fdiv_rn(__fsub_rn(v[i], bias), scale));  // mlxaffine.go:165-173
            q = q < 0.0f ? 0.0f : (q > nbins ? nbins : q);
            codes[i] = (uint32_t)q;
        }
        const int64_t r = e0 / K, c = e0 - r * K;
        if (BITS == 4) {
            uint32_t word = 0;
#pragma unroll
            for (int i = 0; i < 8; i++) word |= codes[i] << (4 * i);
            if (live) packed[e0 / 8] = word;
        } else if (BITS == 8) {
            uint32_t w0 = codes[0] | (codes[1] << 8) | (codes[2] << 16) | (codes[3] << 24);
            uint32_t w1 = codes[4] | (codes[5] << 8) | (codes[6] << 16) | (codes[7] << 24);
            if (live) { packed[e0 / 4] = w0; packed[e0 / 4 + 1] = w1; }
        } else {  // BITS == 2: 16 codes per word, this lane has 8 of them
            uint32_t half = 0;
#pragma unroll
            for (int i = 0; i < 8; i++) half |= codes[i] << (2 * i);
            const uint32_t other = __shfl_xor_sync(0xffffffffu, half, 1);
            if (live && (t8 & 1) == 0) packed[e0 / 16] = half | (other << 16);
        }
        if (live && (c % gs) == 0) {
            const int64_t gi = r * (K / gs) + c / gs;
            scales[gi] = f32_to_bf16_bits(scale);
            biases[gi] = f32_to_bf16_bits(bias);
        }
    }
}

static int grid_for(int64_t work_items, int block) {
    int64_t g = (work_items + block - 1) / block;
    const int64_t cap = 148 * 16;  // a few resident CTAs per SM; the kernels grid-stride
    if (g > cap) g = cap;
    if (g < 1) g = 1;
    return (int)g;
}

static int32_t validate_codec(int64_t N, int64_t K, int bits, int gs, const char* who) {
    if (!(bits == 2 || bits == 4 || bits == 8)) return fail(LTHN_ERR_INVALID, std::string(who) + ": unsupported bits (want 2, 4 or 8)");
    if (N <= 0 || K <= 0) return fail(LTHN_ERR_INVALID, std::string(who) + ": N and K must be positive");
    if (!(gs == 32 || gs == 64 || gs == 128)) return fail(LTHN_ERR_INVALID, std::string(who) + ": group size must be 32, 64 or 128");
    if (K % gs != 0) return fail(LTHN_ERR_INVALID, std::string(who) + ": group size must divide K");
    return LTHN_OK;
}

template <typename Source>
static int32_t launch_quantize(cudaStream_t s, Source src, int64_t N, int64_t K, int bits, int gs, int variant,
                               uint32_t* packed, uint16_t* scales, uint16_t* biases) {
    const int block = 256;
    const int grid = grid_for(N * K / 8, block);
    if (bits == 4) quantize_kernel<4, Source><<<grid, block, 0, s>>>(src, N, K, gs, variant, packed, scales, biases);
    else if (bits == 8) quantize_kernel<8, Source><<<grid, block, 0, s>>>(src, N, K, gs, variant, packed, scales, biases);
    else quantize_kernel<2, Source><<<grid, block, 0, s>>>(src, N, K, gs, variant, packed, scales, biases);
    LTHN_CUDA_TRY(cudaGetLastError());
    return LTHN_OK;
}

}  // namespace lthn

using namespace lthn;

extern "C" {

int32_t lthn_synth_normal_fill(void* stream, uint64_t seed, uint64_t first, int64_t n, float sigma, float* out) {
    clear_error();
    if (n <= 0) return LTHN_OK;
    LTHN_REQUIRE(out != nullptr, "lthn_synth_normal_fill: out is NULL");
    synth_fill_kernel<<<grid_for(n, 256), 256, 0, (cudaStream_t)stream>>>(seed, first, n, synth_scale(sigma), out);
    LTHN_CUDA_TRY(cudaGetLastError());
    return LTHN_OK;
}

int32_t lthn_affine_quantize(void* stream, const float* w, int64_t N, int64_t K, int32_t bits, int32_t gs,
                             int32_t variant, uint32_t* packed, uint16_t* scales, uint16_t* biases) {
    clear_error();
    int32_t rc = validate_codec(N, K, bits, gs, "lthn_affine_quantize");
    if (rc) return rc;
    LTHN_REQUIRE(w && packed && scales && biases, "lthn_affine_quantize: NULL pointer");
    LTHN_REQUIRE(((uintptr_t)w & 15) == 0, "lthn_affine_quantize: w must be 16-byte aligned");
    return launch_quantize((cudaStream_t)stream, MemSource{w}, N, K, bits, gs, variant, packed, scales, biases);
}

int32_t lthn_synth_affine_weight(void* stream, uint64_t seed, float sigma, int64_t N, int64_t K, int32_t bits,
                                 int32_t gs, int32_t variant, uint32_t* packed, uint16_t* scales, uint16_t* biases) {
    clear_error();
    int32_t rc = validate_codec(N, K, bits, gs, "lthn_synth_affine_weight");
    if (rc) return rc;
    LTHN_REQUIRE(packed && scales && biases, "lthn_synth_affine_weight: NULL pointer");
    return launch_quantize((cudaStream_t)stream, SynthSource{seed, synth_scale(sigma), K, K, 0, 0}, N, K, bits, gs, variant,
                           packed, scales, biases);
}

// Rows [row0,row0+N) x columns [col0,col0+K) of the synthetic [*,Kfull] tensor, 4 bit, group 64.
int32_t lthn_synth_affine_weight_shard(void* stream, uint64_t seed, float sigma, int64_t N, int64_t K, int64_t row0,
                                       int64_t col0, int64_t Kfull, uint32_t* packed, uint16_t* scales,
                                       uint16_t* biases) {
    clear_error();
    int32_t rc = validate_codec(N, K, 4, 64, "lthn_synth_affine_weight_shard");
    if (rc) return rc;
    LTHN_REQUIRE(packed && scales && biases && col0 % 64 == 0 && col0 + K <= Kfull, "lthn_synth_affine_weight_shard: bad shard");
    return launch_quantize((cudaStream_t)stream, SynthSource{seed, synth_scale(sigma), K, Kfull, row0, col0}, N, K, 4, 64, 0,
                           packed, scales, biases);
}

static int32_t dequant_any(void* stream, const uint32_t* packed, const uint16_t* scales, const uint16_t* biases,
                           int64_t N, int64_t K, int32_t bits, int32_t gs, void* out, bool bf16, const char* who) {
    clear_error();
    int32_t rc = validate_codec(N, K, bits, gs, who);
    if (rc) return rc;
    LTHN_REQUIRE(packed && scales && biases && out, "dequantize: NULL pointer");
    const int block = 256;
    const int grid = grid_for(N * K * bits / 32, block);
    cudaStream_t s = (cudaStream_t)stream;
#define LTHN_DQ(B)                                                                                         \
    if (bf16) dequant_kernel<B, true><<<grid, block, 0, s>>>(packed, scales, biases, N, K, gs, out);      \
    else dequant_kernel<B, false><<<grid, block, 0, s>>>(packed, scales, biases, N, K, gs, out);
    if (bits == 4) { LTHN_DQ(4) } else if (bits == 8) { LTHN_DQ(8) } else { LTHN_DQ(2) }
#undef LTHN_DQ
    LTHN_CUDA_TRY(cudaGetLastError());
    return LTHN_OK;
}

int32_t lthn_affine_dequantize(void* stream, const uint32_t* packed, const uint16_t* scales, const uint16_t* biases,
                               int64_t N, int64_t K, int32_t bits, int32_t gs, float* out) {
    return dequant_any(stream, packed, scales, biases, N, K, bits, gs, out, false, "lthn_affine_dequantize");
}
int32_t lthn_affine_dequantize_bf16(void* stream, const uint32_t* packed, const uint16_t* scales,
                                    const uint16_t* biases, int64_t N, int64_t K, int32_t bits, int32_t gs,
                                    uint16_t* out) {
    return dequant_any(stream, packed, scales, biases, N, K, bits, gs, out, true, "lthn_affine_dequantize_bf16");
}

}  // extern "C"
