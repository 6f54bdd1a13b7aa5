// Layer-list models: a decoder described by a list of layers, each a token mixer (of several kinds) and an optional
// feed-forward block, over dense bf16 / f32 tensors. Internal launch interfaces between the graph (layered.cu), the
// dense products (dense.cu) and the mixer kernels (mixers.cu). The llama graph over GGUF blocks is engine.cu.
//
// A step is a RAGGED batch: `n_seg` segments (one per sequence taking part), segment s brings seg_len[s] consecutive
// tokens of the sequence in slot seg_slot[s] starting at position seg_pos0[s]; all T tokens are concatenated. Prompt
// portions and single decoded tokens are the same thing. Every kernel below reads this description from device memory.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

struct b2_engine;

namespace b2 {

struct RaggedDev {             // device pointers, valid for one step
    const int* tok_id;         // [T] token ids
    const int* tok_seg;        // [T] segment of each token
    const int* tok_pos;        // [T] position inside its sequence
    const int* seg_slot;       // [n_seg]
    const int* seg_start;      // [n_seg] first row of the segment
    const int* seg_len;        // [n_seg]
    const int* seg_pos0;       // [n_seg] position of the segment's first token
    const int* tile_seg;       // [n_tiles] tiles of up to 64 consecutive rows of one segment: its segment ...
    const int* tile_row0;      // ... and its first row
    int T, n_seg, n_tiles;
};

// ---------------------------------------------------------------- dense products (dense.cu)
// Y[t][n] = epi(sum_k X[t][k] * W[n][k] (+ bias[n])), X f32 [T][ldx], W [N][K] (bf16 or f32), Y f32 [T][ldy].
// Each output element is one fixed-order sum over k: a row's result does not depend on what else is in the batch.
enum DenseEpi { EPI_NONE = 0, EPI_BIAS = 1, EPI_BIAS_RELU2 = 2 };
struct DenseArgs {
    const float* x; int ldx;
    const void* w; int w_type;      // T_BF16 or T_F32 (quant_blocks.cuh ids)
    const float* bias;              // f32 [N] or null
    float* y; int ldy;
    int T, N, K;
    int epi;
    bool exact;                     // true: 32-bit multiply-adds (no tensor cores, inputs not rounded)
    __nv_bfloat16* xb;              // scratch [T][K] for X rounded to bf16 (large tensor-core steps); null: not available
};
cudaError_t dense_launch(const DenseArgs& a, cudaStream_t s);

// ---------------------------------------------------------------- mixers and norms (mixers.cu)
cudaError_t embed_ragged_launch(const void* table, int w_type, int W, const int* tok_id, int T, float* x, cudaStream_t s);
// gather rows: y[i] = x[rows[i]]
cudaError_t gather_rows_launch(const float* x, int W, const int* rows, int n, float* y, cudaStream_t s);

// Post-sum layer norm: x[t] = LN(alpha * x[t] + y[t]) * w with
//   y = a                      (b == nullptr)
//   y = (rms(a) * wa + rms(b) * wb) / 2   (two branches, each RMS-normed over the width first)
cudaError_t postsum_norm_launch(float* x, const float* a, const float* wa, const float* b, const float* wb, const float* w,
                                float alpha, float eps, int W, int T, cudaStream_t s);
// plain layer norm without bias: y[t] = LN(x[t]) * w
cudaError_t layer_norm_launch(const float* x, const float* w, float eps, int W, int T, float* y, cudaStream_t s);

struct RotaryTable {           // cos and sin of position * frequency (frequencies already blended, magnitude factor folded
    const float* cos;          // in), [n_ctx][rot_dims / 2] each, built on the host in double precision
    const float* sin;
    int rot_dims;
};
struct WindowAttnArgs {
    const float* proj; int ldp; int q_off, k_off;     // projection rows: q at q_off [H*d], k at k_off [G*d]
    const float* q_norm_w; const float* k_norm_w;     // [d]
    RotaryTable rot;
    void* k_pool; void* v_pool; int cache_f32;        // pages [page][G][block_tokens][d]; bf16 or f32
    int* const* block_tables;                         // [slot] -> page table
    int block_tokens;
    int H, G, d;
    int window, keep_first;
    float scale, eps;
    float* q_rot;              // scratch [T][H*d]
    float* out;                // [T][H*d]
    float* split_scratch;      // few-token steps: partial (max, sum, output) per key range, [T][H][splits][d + 2]
    int split_capacity;        // floats in split_scratch
};
// norm + rotate q and k, store k (rotated) and v (= k as projected) into the pages
cudaError_t window_attn_store_launch(const WindowAttnArgs& a, const RaggedDev& r, cudaStream_t s);
// softmax attention of every step token over the visible cached keys of its sequence
cudaError_t window_attn_launch(const WindowAttnArgs& a, const RaggedDev& r, cudaStream_t s);

struct ScanArgs {              // selective scan (Mamba)
    const float* proj; int ldp; int x_off, z_off;     // W_in output rows: x at x_off [inner], z at z_off [inner]
    const float* conv_w; const float* conv_b; int taps;   // [inner][taps], [inner]
    float* conv_state;         // [slot][inner][taps-1] last inputs, newest last
    float* xc;                 // [T][inner] convolved + SiLU
    const float* xproj; int ldx; int R, N;            // W_x output rows: dt [R] | B [N] | C [N]
    const float* dt_raw;       // [T][inner] W_dt dt (bias not yet added)
    const float* dt_bias; const float* A_log; const float* D;
    float* ssm_state;          // [slot][inner][N]
    float* y;                  // [T][inner] gated output
    int inner;
};
cudaError_t scan_conv_launch(const ScanArgs& a, const RaggedDev& r, cudaStream_t s);
cudaError_t scan_recurrence_launch(const ScanArgs& a, const RaggedDev& r, cudaStream_t s);

struct MatrixMemArgs {         // mLSTM
    const float* proj; int ldp; int q_off, k_off, v_off, g_off, i_off, f_off;
    const float* i_bias; const float* f_bias; const float* norm_w;
    int H, d, dv;
    float cap, eps;
    float* S; float* n; float* m;      // per slot: [H][d][dv], [H][d], [H]
    float* o_raw;              // [T][H*dv] scratch: memory read-out before the head norm
    float* out;                // [T][H*dv]
};
cudaError_t matrix_mem_launch(const MatrixMemArgs& a, const RaggedDev& r, cudaStream_t s);

// ---------------------------------------------------------------- graph (layered.cu)
struct LayeredModel;
int layered_finalize(b2_engine* e);
void layered_destroy(b2_engine* e);
int layered_seq_reset(b2_engine* e, int slot);

}  // namespace b2
