// qmv_i8.cu — planning and dispatch of the integer tensor-core affine_qmv kernel
// (kernel and its description: qmv_i8_kernel.cuh; instantiations: qmv_i8_inst*.cu).
#include "common.cuh"
#include "qmv.hpp"

#include <algorithm>

namespace lthn {

struct I8Args;
template <int J>
int32_t launch_i8_w(cudaStream_t st, const I8Args& a, const I8Plan& p, int M, int fuse);
template <int J>
int32_t launch_i8_b8(cudaStream_t st, const I8Args& a, const I8Plan& p, int M, int fuse);
int32_t i8_launch_args(cudaStream_t st, const QmvCall& c, const I8Plan& p);

// ---- host side --------------------------------------------------------------------

LTHN_HIDDEN int g_i8_stg = 0;  // ring-stage override: zero in the product library (setter: test_hooks.cu)
// dynamic shared memory a block may ask for (the SM has 227 KB for one block)
static const size_t kI8MaxSmem = 224 * 1024;
static const int kI8J[] = {1, 2, 3, 4, 6, 7, 8, 9, 12, 16, 18, 21};

static bool i8_plan_slice(int64_t N, int Gs, int ks, int M, int fuse, int force_w, bool has_norm, I8Plan* p, int bits = 4) {
    // (J, W): W consumer warps of J groups each. Measured on B200: a long stream (many row blocks
    // per SM) runs fastest with few warps per block and many blocks per SM (less hand-off per row
    // block, more independent pipelines: 5.9 TB/s with 4 warps against 4.4 with 12 on the 340 MB
    // lm_head); a small matrix, where each block sees only a few row blocks, finishes sooner with
    // the groups spread over as many warps as possible.
    const int out_rows = fuse == 2 ? 8 : 16;  // output rows per row block (fuse 2: 8 gate + 8 up rows)
    const double per_sm = (double)(N / out_rows) * ks / 148.0;
    // measured crossover: about four row blocks per SM; a fused norm prologue is work per warp that
    // many warps finish sooner, so it moves the crossover up
    const int target = per_sm < (has_norm ? 16.0 : 4.0) ? 16 : 4;
    int J = 0, W = 0, best = -1;
    for (int cand : kI8J) {
        if (Gs % cand) continue;
        const int w = Gs / cand;
        if (w < 1 || w > 16) continue;
        if (bits == 8 && ((cand != 2 && cand != 3 && cand != 4 && cand != 6 && cand != 9 && cand != 12) || (cand > 9 && w > 8))) continue;
        if (cand > 9 && w > 8) continue;  // many groups per warp only in small blocks (registers)
        // the five-blocks-per-SM build of the 4-warp class holds 72 registers: the digit fragments of
        // more than 9 groups (4 registers each) do not fit and spill (K = 5376 as 4 x 21 groups
        // measured 94 us for the 130 MB gate/up pair, 1.4 TB/s)
        if (cand > 9 && w <= 4) continue;
        int score = 1000 - 10 * std::abs(w - target) + (target >= 8 ? w : -w);
        if (force_w > 0) score = (w == force_w) ? 5000 : -1;
        if (score > best) { best = score; J = cand; W = w; }
    }
    if (best < 0) return false;
    const int sets = fuse == 1 ? 2 : 1;
    const int rsw = Gs * 2 * bits;  // words of codes per row (slice)
    const int padw = ((8 - rsw % 32) + 32) % 32;
    const int RS = (rsw + padw) * 4;
    const int RB = 16;
    const int nblocks = (int)((N + out_rows - 1) / out_rows);
    const size_t sb = ((size_t)RB * Gs * 2 + 15) / 16 * 16;
    const size_t stage = sets * ((size_t)RB * RS + 2 * sb);
    for (int stg = g_i8_stg >= 2 && g_i8_stg <= 4 ? g_i8_stg : 2; stg >= 2; stg--) {
        const size_t part_bytes = (size_t)2 * stg * W * sets * RB * M * 4;
        const size_t bs_off = 512 + part_bytes;
        const size_t stage_off = (bs_off + (size_t)W * (M * 192 + J * 32) + 127) / 128 * 128;
        const size_t smem = stage_off + (size_t)stg * stage;
        if (smem > kI8MaxSmem) continue;
        p->J = J; p->W = W; p->RT = 1; p->stg = stg; p->RS = RS; p->nblocks = nblocks;
        p->threads = (W + 1) * 32;
        p->bs_off = (int)bs_off; p->stage_off = (int)stage_off;
        p->ks = ks; p->Gs = Gs; p->fuse = fuse;
        p->smem = smem;
        return true;
    }
    return false;
}

bool i8_plan(int64_t N, int64_t K, int M, int fuse, int force_ks, int force_w, I8Plan* p, int max_slices, bool has_norm) {
    if (M < 1 || M > 2 || K % 64 != 0 || N < 16 || N % 16 != 0) return false;
    const int G = (int)(K / 64);
    // GeGLU pairs: long rows use the interleaved row block (half the shared memory per stage);
    // measured: K=5376 42 -> 24 us at N=21504, K=2304 slightly slower than two full sets
    if (fuse) fuse = K >= 4096 ? 2 : 1;
    // Whole rows whenever a 16-row block of the whole K fits the shared-memory ring (K <= 10752).
    // K slices (partial sums + a summing pass) exist for longer rows but were measured slower than
    // the dp4a kernel on the shapes tried (K = 14336..21504), and
    // slower than whole rows on small matrices, so the dispatcher only uses them when asked to
    // (max_slices > 1). A GeGLU epilogue needs whole rows.
    if (force_ks <= 1 && i8_plan_slice(N, G, 1, M, fuse, force_w, has_norm, p)) return true;
    if (fuse || has_norm || max_slices <= 1) return false;  // a GeGLU epilogue and a norm prologue need whole rows
    int best_ks = 0, best_d = 1 << 30;
    for (int ks : {2, 3, 4, 6, 8}) {
        if (ks > max_slices || G % ks) continue;
        if (force_ks > 1 && ks != force_ks) continue;
        const int Gs = G / ks;
        if ((Gs & 1) || (G & 1) || Gs < 16) continue;
        I8Plan q;
        if (!i8_plan_slice(N, Gs, ks, M, 0, force_w, false, &q)) continue;
        const int d = std::abs(Gs - 48);
        if (d < best_d) { best_d = d; best_ks = ks; *p = q; }
    }
    return best_ks != 0;
}

// 8-bit codes, one or two rows: whole rows while a 16-row block fits the ring (K <= ~5376), else K slices with
// partial sums. Measured on B200 (one row): 2304 x 9216 takes 15.0 / 15.4 / 14.0 / 10.4 / 10.9 us with 2 / 3 / 4 /
// 6 / 8 slices, 5376 x 21504 59 / 61 / 46 us with 4 / 6 / 8 - many short slices (several blocks per SM, all of
// the matrix in flight at once) beat few long ones, so the slice count whose slices are nearest 24 groups wins.
// A GeGLU pair (fuse) or a fused norm prologue needs whole rows; rows of 2048 codes and more take the
// interleaved 8 + 8 row block, as 4-bit rows of the same byte length do.
bool i8_plan_b8(int64_t N, int64_t K, int M, I8Plan* p, int force_ks, int force_w, int fuse, bool has_norm) {
    if (M < 1 || M > 2 || K % 64 != 0 || N < 16 || N % 16 != 0) return false;
    const int G = (int)(K / 64);
    if (fuse) fuse = K >= 2048 ? 2 : 1;
    if (force_ks <= 1 && i8_plan_slice(N, G, 1, M, fuse, force_w, has_norm, p, 8)) return true;
    if (fuse || has_norm) return false;
    int best_ks = 0, best_d = 1 << 30;
    for (int ks : {2, 3, 4, 6, 8}) {
        if (G % ks || (force_ks > 1 && ks != force_ks)) continue;
        const int Gs = G / ks;
        if ((Gs & 1) || (G & 1) || Gs < 8) continue;
        I8Plan q;
        if (!i8_plan_slice(N, Gs, ks, M, 0, force_w, false, &q, 8)) continue;
        const int d = std::abs(Gs - 24);
        if (d < best_d) { best_d = d; best_ks = ks; *p = q; }
    }
    return best_ks != 0;
}

bool qmv_can_fuse_norm(int64_t N, int64_t K, int M, bool geglu, int bits) {
    I8Plan p;
    if (bits == 8) return i8_plan_b8(N, K, M, &p, 0, 0, geglu ? 1 : 0, true);
    return i8_plan(N, K, M, geglu ? 1 : 0, 0, 0, &p, 1, true);
}

int32_t i8_launch(cudaStream_t st, const QmvCall& c, const I8Plan& p) { return i8_launch_args(st, c, p); }

}  // namespace lthn
