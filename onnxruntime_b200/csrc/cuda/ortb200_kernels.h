// C ABI of the sm_100a kernel library (libortb200_kernels.so).
//
// Every function takes raw device pointers plus a cudaStream_t and returns 0
// on success or a negative code when the arguments are rejected on the host
// (nothing is launched in that case).  Device-side problems (a bounded wait
// that ran out) are reported through the int status word the caller passes;
// 0 means the launch completed normally.
//
// The library does not depend on PyTorch; the torch extension and ctypes-based
// tests both call it through these symbols.
#pragma once
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef void* ortb200_stream_t;  // cudaStream_t

enum ortb200_dtype { ORTB200_F16 = 0, ORTB200_BF16 = 1, ORTB200_F32 = 2, ORTB200_F8E4M3 = 3, ORTB200_Q4 = 4, ORTB200_F8W = 5 };

enum ortb200_act {
  ORTB200_ACT_NONE = 0,
  ORTB200_ACT_GELU = 1,      // erf form
  ORTB200_ACT_FASTGELU = 2,  // tanh form
  ORTB200_ACT_RELU = 3,
  ORTB200_ACT_SILU = 4,
  ORTB200_ACT_SWIGLU = 5,    // silu(W1 x) * (W2 x); W2 rows start `dual_offset` rows after W1 rows
  ORTB200_ACT_QUICKGELU = 6,
};

// out[M, N] = act(alpha * X[M, K] * W[N, K]^T + bias[N]) + residual[M, N]
// X and W are row-major with K contiguous (K % 8 == 0, 16-byte aligned bases).
// tcgen05 / TMEM tensor-core GEMM; weights ride the 128-lane M side of the MMA
// and tokens the N side, so decode (M = 1..16) streams W once at HBM speed and
// prefill uses 128x{128,256} tiles.  `workspace` holds split-K partial tiles and
// tile counters; ortb200_gemm_workspace_bytes() gives an upper bound for a
// problem.  The counters must be zero before the first launch (the kernel leaves
// them zero again).
typedef struct {
  const void* x;        // [M, K]
  const void* w;        // [N_total, K]; N rows used for the first operand
  void* out;            // [M, ldo]
  const void* bias;     // [N] or null, same dtype as out
  const void* residual; // [M, ldr] or null, same dtype as out
  int64_t ldo, ldr;
  int M, N, K;
  int w_rows;           // total rows in w (>= N, or >= dual_offset + N for SWIGLU)
  int dual_offset;      // SWIGLU only
  int dtype;            // ortb200_dtype of x, w, out, bias, residual (F16 or BF16)
  int act;              // ortb200_act
  float alpha;
  void* workspace;      // device scratch, may be null when splits == 1 is forced
  int64_t workspace_bytes;
  int* status;          // device int, may be null
  int force_splits;     // 0 = heuristic
  int force_bn;         // 0 = heuristic; else 16/32/64/128/256
  int use_pdl;          // launch with programmatic stream serialization
  // Fused all-reduce (row-parallel linear): when world > 1 the kernel sums the partial products of all ranks
  // itself.  Each epilogue thread pushes its fp32 partial sums into every rank's symmetric workspace as 64-bit
  // words (value in the low half, the launch's epoch in the high half) with plain peer stores, then polls (bounded)
  // the words of all source ranks in its own workspace until they carry the epoch, adds them in rank order, and
  // applies bias / residual as usual.  No fence, flag or barrier is involved: one NVLink store latency per GEMM.
  // Requires M <= 64, ldo == N, no dual (SwiGLU) epilogue.
  // peers[i] is rank i's workspace base as mapped into this process; the layout is
  //   [0, 256 KiB)    epoch word (offset 0), done counter (offset 4), polling limit override (offset 8, 0 = default),
  //                   rest reserved
  //   [256 KiB, bytes / 2)  staging[2][world][slot] 64-bit words, slot = (bytes / 2 - 256 KiB) / (2 * world * 8) >= M * ldo
  //   [bytes / 2, bytes)    used by ortb200_symm_collective
  // Two staging halves alternate by epoch parity, so a rank that runs one launch ahead never overwrites words a
  // slower rank still has to read.  The workspace must be zero before the first launch, and all ranks must launch
  // the same sequence of fused GEMMs.
  int world;
  int rank;
  void* peers[8];
  int64_t symm_bytes;
  // Operand type when it differs from `dtype`: ORTB200_F8E4M3 = x and w hold e4m3 bytes (K a multiple of 16) and
  // the tensor cores run in their 8-bit mode; out / bias / residual keep `dtype`, `alpha` carries the product of
  // the per-tensor scales.  0 = operands are of `dtype`.
  int in_dtype;
  // Fused RMS normalisation of x (decode-shaped problems, M <= 64, only): when rms_eps > 0 the kernel computes
  // out = act(alpha * (x @ w^T) / rms(x) + bias) + residual with rms(x)[m] = sqrt(mean_k x[m, k]^2 + rms_eps);
  // the caller folds the norm's gamma into w (w[n, k] *= gamma[k]).  Larger M returns -14: normalise first.
  float rms_eps;
  // in_dtype == ORTB200_Q4 (decode-shaped problems, M <= 64): w is the tile-blob array that the caller builds once
  // from MatMulNBits weights (layout below); the kernel fetches one contiguous blob per (weight tile, k-block) and
  // expands the nibbles to `dtype` in shared memory on their way to the tensor cores.  K a multiple of 64.
  //   blob(tile t, k-block kb) at byte ((t * K / 64) + kb) * 4864:
  //     [0, 4096)    row r (weight row 128 t + r) at r * 32: the 64 nibbles of the k-block, re-arranged per 32-bit word
  //                  by ortb200_nbits_prepack
  //     [4096, 4608) row r at r * 4: the scales of elements [0, 32) and [32, 64) of the k-block, in `dtype`
  //     [4608, 4864) row r at r * 2: their zero points, one byte each (8 when the model has none)
  //   rows beyond N are zero.  W[n, k] = (q - zp) * scale.
  // in_dtype == ORTB200_F8W (decode-shaped problems, M <= 64): weight-only fp8.  w is a tile-blob array like the 4-bit
  // one: blob(tile t, k-block kb) at byte ((t * K / 64) + kb) * 8704 holds [0, 8192) row r at r * 64: the 64 e4m3 bytes
  // W[128 t + r, 64 kb ... 64 kb + 63], and [8192, 8704) row r at r * 4: the fp32 scale of that row and k-block.
  // W[n, k] = e4m3(byte) * scale.  The kernel expands to `dtype` on the way to the tensor cores.  K a multiple of 64.
  int force_tile_rows;  // 0 / 128 = 128-weight-row CTA tiles; 256 = 256-row tiles in the large-M kernel (M > 128);
                        // 512 = pairs of CTAs on 256 x 256 tiles (cta_group::2 kernel)
  // Prompt-sized fused all-reduce (world > 1, M > 64) with NVLS: the multicast address of the symmetric workspace.  The
  // reduction kernel then replicates the sums with one multimem.st per 16 bytes instead of a store to every peer.
  // Null: peer stores only.
  void* mc_ptr;
  // Optional device scalar (fp32) multiplied into alpha by the kernel: scales that only exist on the device (GemmFloat8 with
  // runtime scale inputs) need no host read.  fp8 operand mode only; null otherwise.
  const float* alpha_dev;
} ortb200_gemm_args;

int ortb200_gemm(const ortb200_gemm_args* args, ortb200_stream_t stream);

// Grouped GEMM (mixture of experts): rows of x are sorted by expert; a device-side tile list says which expert's
// weights multiply which row range, so no count ever travels to the host:
//   out[r, :] = act(x[r, :] @ w[e]^T + bias[e]) for first_row <= r < end_row of every tile {e, first_row, end_row, -}.
// Tiles cover at most tile_rows rows each.  tile_rows in {16, 32, 64}: one CTA per (weight tile, token tile), the
// grid has max_tiles rows of CTAs and the CTAs beyond *num_tiles leave at once.  tile_rows in {128, 256}: the
// persistent large-tile kernel walks the list (SWIGLU needs 128).  w is [num_experts * w_rows_per_expert, K]; with act == SWIGLU the gate rows
// of expert e start at e * w_rows_per_expert and the up rows dual_offset rows later (N = rows of each half).
typedef struct {
  const void* x;          // [rows, K]
  const void* w;
  void* out;              // [rows, N]
  const void* bias;       // optional [num_experts, N]
  const void* tile_info;  // int4 per tile (16-byte aligned)
  const int* num_tiles;   // device scalar
  int rows, N, K;
  int num_experts, w_rows_per_expert, dual_offset;
  int tile_rows, max_tiles;
  int dtype, act;
  int* status;
  int use_pdl;
} ortb200_gemm_grouped_args;
int ortb200_gemm_grouped(const ortb200_gemm_grouped_args* args, ortb200_stream_t stream);

// ---------------------------------------------------------------------------
// A chain of decode-shaped GEMMs (M <= 16 token rows) in one persistent launch: stage s computes
//   y_s[M, N_s] = act_s((x_s[M, K_s] @ W_s[N_s, K_s]^T) / rms(x_s) + bias_s) + residual_s      with x_0 = x, x_{s+1} = y_s
// so K_{s+1} must equal N_s.  One CTA per SM walks all stages; the weight stream of stage s + 1 runs while stage s
// drains, which is what a sequence of separate launches cannot do (gemm_chain.cu).  K_s must be a multiple of 64.
#define ORTB200_CHAIN_MAX_STAGES 4
typedef struct {
  const void* w;         // [w_rows, K], K contiguous; with rms_eps > 0 the caller has folded the norm's gamma into it
  void* out;             // [M, N] contiguous (also the next stage's input)
  const void* bias;      // [N] or null
  const void* residual;  // [M, ldr] or null; ignored when residual_stage >= 0
  int64_t ldr;
  int N, K, w_rows;
  int dual_offset;       // act == SWIGLU: up rows start dual_offset rows after the gate rows
  int act;               // ortb200_act
  float rms_eps;         // > 0: divide by rms of the stage's input rows (not for stage 0, not with all_reduce)
  int residual_stage;    // >= 0: the residual is the output of that earlier stage of this chain; -1 = use `residual`
  int all_reduce;        // world > 1: sum the products of all ranks before bias / activation / residual
} ortb200_chain_stage;

typedef struct {
  const void* x;         // [M, K_0]
  int M;                 // 1..16
  int num_stages;        // 1..ORTB200_CHAIN_MAX_STAGES
  int dtype;             // F16 or BF16 (everything: x, weights, outputs, bias, residual)
  ortb200_chain_stage stage[ORTB200_CHAIN_MAX_STAGES];
  void* workspace;       // ortb200_gemm_chain_workspace_bytes() bytes, zero before the first launch, left zero
  int64_t workspace_bytes;
  int* status;           // device int, may be null
  int use_pdl;
  int prefetch_items;    // how many (tile, k-block) items beyond its shared-memory ring a CTA asks the L2 for (0 = none)
  int max_ctas;          // 0 = one CTA per SM
  // tensor parallelism, as in ortb200_gemm_args (same symmetric workspace layout and epoch counter)
  int world, rank;
  void* peers[8];
  int64_t symm_bytes;
  void* trace;           // optional device buffer of gridDim x 32 uint64: %globaltimer stamps of the launch's phases (profiling)
} ortb200_gemm_chain_args;
int64_t ortb200_gemm_chain_workspace_bytes(void);
int ortb200_gemm_chain(const ortb200_gemm_chain_args* args, ortb200_stream_t stream);
int64_t ortb200_gemm_workspace_bytes(int M, int N, int K, int act);

// All-gather -> GEMM as one kernel: x is sharded by rows over the ranks (this rank holds x_local [rows_local, K]) and
// out [world * rows_local, N] = act(concat over ranks of x_local @ w^T + bias) for this rank's w [N, K].  Four extra
// warps of every CTA push the shard into the other ranks' symmetric workspaces with peer stores while the tensor-core
// warps start on the rank's own rows; the tiles of another rank's rows wait (bounded, status word) for that rank's one
// flag and are read from local memory by TMA, so every remote row crosses NVLink once.  The call counts as one step
// of the collectives' epoch (all ranks must issue the same sequence of collective calls); the gather areas are the
// result areas of ortb200_symm_collective's workspace halves, so world * rows_local * K * 2 bytes must fit in
// symm_bytes / 8 (ortb200_allgather_gemm_max_rows).  K a multiple of 8, 16-bit types, pointers 16-byte aligned.
typedef struct {
  const void* x_local;
  const void* w;
  const void* bias;      // optional [N]
  void* out;
  int rows_local, N, K;
  int dtype, act;        // act: NONE / GELU / FASTGELU / RELU / SILU / QUICKGELU
  int world, rank;
  void* peers[8];
  int64_t symm_bytes;
  int* status;
  int use_pdl;
} ortb200_allgather_gemm_args;
int ortb200_allgather_gemm(const ortb200_allgather_gemm_args* args, ortb200_stream_t stream);
int64_t ortb200_allgather_gemm_max_rows(int world, int K, int64_t symm_bytes);
// Byte offsets inside a symmetric workspace that the kernel above uses (for tests that stand in for a peer):
// the gather area of `parity`, and the flag word that source rank `src` raises.
int64_t ortb200_allgather_gemm_area_offset(int64_t symm_bytes, int parity);
int64_t ortb200_allgather_gemm_flag_offset(int src);
// Number of kernels one ortb200_gemm call launches (always 1).
int ortb200_gemm_last_config(int* bn, int* splits, int* stages);

// ---------------------------------------------------------------------------
// (Skip)LayerNorm / (Skip)SimplifiedLayerNorm.  out = norm(x + skip + bias) * gamma (+ beta);
// sum_out (optional) receives x + skip + bias, the residual stream.  All pointers 16-byte aligned,
// hidden * sizeof(T) a multiple of 16, hidden <= 16 * 256 * (16 / sizeof(T)).
typedef struct {
  const void* x;
  const void* skip;   // optional
  const void* bias;   // optional [hidden]
  const void* gamma;  // [hidden]
  const void* beta;   // optional [hidden]
  void* out;
  void* sum_out;      // optional
  int64_t rows;
  int hidden;
  float epsilon;
  int simplified;     // 1 = RMS form (no mean subtraction, no beta)
  int dtype;
} ortb200_norm_args;
int ortb200_norm(const ortb200_norm_args* args, ortb200_stream_t stream);

// EmbedLayerNormalization: out[b, s, :] = LayerNorm(word[ids] + pos[position] + seg[segment]) * gamma + beta.
// ids are int32 or int64 (id_bytes 4 / 8); position_ids optional ([B, S], or [1, S] with position_broadcast = 1;
// absent = 0 .. S - 1); segment ids / table optional.  hidden * element size must be a multiple of 16, at most 4096
// elements of 16 bits (2048 of 32).  An id outside its table sets *status to the bad-argument code and reads row 0.
typedef struct {
  const void* input_ids;
  const void* segment_ids;
  const void* position_ids;
  const void* word_emb;
  const void* pos_emb;
  const void* segment_emb;
  const void* gamma;
  const void* beta;
  void* out;           // [B, S, hidden]
  void* sum_out;       // optional [B, S, hidden]: the embedding sum before normalisation
  int B, S, hidden;
  int word_rows, pos_rows, seg_rows;
  int id_bytes, position_broadcast;
  float epsilon;
  int dtype;
  int* status;         // optional device int
} ortb200_embed_layernorm_args;
int ortb200_embed_layernorm(const ortb200_embed_layernorm_args* args, ortb200_stream_t stream);

// ---------------------------------------------------------------------------
// GroupQueryAttention, step 1: split packed QKV, apply rotary embedding to Q and K, append K/V to the cache.
// Caches are [B, Nk, Smax, H].  Position of token s of batch b: position_ids[b, s] when given, else
// past_len(b) + s with past_len(b) = first_prompt ? 0 : seqlens_k[b] + 1 - S.
typedef struct {
  const void* qkv;             // packed [B, S, (N + 2 Nk) H], or Q [B, S, N H] when k / v are given
  const void* k;               // optional [B, S, Nk H]
  const void* v;               // optional [B, S, Nk H]
  void* q_out;                 // [B, S, N, H]
  void* k_cache;
  void* v_cache;
  const int* seqlens_k;        // [B], total length - 1
  const void* cos_cache;       // [max_pos, rot_dim / 2] (same dtype); null when do_rotary == 0
  const void* sin_cache;
  const int64_t* position_ids; // optional [B, S]
  int B, S, N, Nk, H, Smax;
  int rot_dim;                 // 0 = H
  int interleaved;
  int first_prompt;
  int do_rotary;
  int dtype;
  int use_pdl;                 // launch with programmatic stream serialization (overlaps the previous kernel's tail)
  int cos_rows;                // rows of cos_cache / sin_cache; positions are clamped to it (0 = not checked)
} ortb200_gqa_prep_args;
int ortb200_gqa_prep(const ortb200_gqa_prep_args* args, ortb200_stream_t stream);

// PagedAttention, step 1 (packed tokens [T, ...]): token t belongs to the sequence b with
// cu_seqlens[b] <= t < cu_seqlens[b + 1] and sits at position past_seqlens[b] + t - cu_seqlens[b].  Q and K are rotated
// at that position; K / V go to cache slot slot_mapping[t] (negative = skip) or, without a slot mapping, to
// block_table[b, pos / block_size] * block_size + pos % block_size.  Caches are [num_blocks, block_size, Nk, H].
typedef struct {
  const void* qkv;             // packed [T, (N + 2 Nk) H], or Q [T, N H] when k / v are given
  const void* k;
  const void* v;
  void* q_out;                 // [T, N, H]
  void* k_cache;
  void* v_cache;
  const int* cu_seqlens;       // [B + 1]
  const int* past_seqlens;     // [B]
  const int* block_table;      // [B, max_blocks]
  const int64_t* slot_mapping; // optional [T]
  const void* cos_cache;
  const void* sin_cache;
  int T, B, N, Nk, H;
  int block_size, max_blocks, num_blocks;
  int rot_dim, interleaved, do_rotary, dtype;
  int* status;                 // device int, may be null: a block index outside the table is reported here
  int cos_rows;                // rows of cos_cache / sin_cache; positions are clamped to it (0 = not checked)
} ortb200_paged_prep_args;
int ortb200_paged_prep(const ortb200_paged_prep_args* args, ortb200_stream_t stream);

// GroupQueryAttention, decode step (one query token per sequence): split-KV attention over the cache.
// q [B, N, H]; attends to cache positions [max(0, total - window), total) with total = seqlens_k[b] + 1.
// workspace: ortb200_gqa_decode_workspace_bytes(); its first 64 KiB (counters) must be zero before the first
// launch and is left zero.  H must be 64 or 128.
typedef struct {
  const void* q;
  const void* k_cache;
  const void* v_cache;
  const int* seqlens_k;
  const void* head_sink;  // optional [N], same dtype
  void* out;              // [B, N H]
  void* workspace;
  int64_t workspace_bytes;
  int B, N, Nk, H, Smax;
  int splits;             // 0 = heuristic
  int window;             // <= 0: none
  float scale;            // 0 = 1/sqrt(H)
  float softcap;
  int dtype;
  int use_pdl;
  int* status;            // device int, may be null (bounded waits report here)
  // Paged cache (PagedAttention): when block_table is given, k_cache / v_cache are [num_blocks, block_size, Nk, H]
  // and key j of sequence b lives in block block_table[b * max_blocks + j / block_size]; Smax is then only the
  // upper bound of the sequence length used to size the split-KV grid.
  const int* block_table;
  int block_size;
  int max_blocks;
  // Fused step 1 (replaces ortb200_gqa_prep for one-token steps): when qkv is given, q is ignored; query, key and
  // value of the new token are read from the packed projection output qkv [B, (N + 2 Nk) H], rotated at position
  // seqlens_k[b] (cos / sin caches [max_pos, H / 2], full-width rotary) and the new key / value are written to cache
  // position seqlens_k[b] by the kernel itself.
  const void* qkv;
  const void* cos_cache;
  const void* sin_cache;
  int do_rotary;
  int rotary_interleaved;
  int num_blocks;         // paged cache: blocks in the pool (needed by the tensor-core kernel; 0 = unknown)
  int algo;               // 0 = pick, 1 = CUDA-core split-KV kernel, 2 = tcgen05 kernel (error if unsupported)
  // Optional hint (tcgen05 kernel): device memory the next kernel will stream (the output projection's weights).  The
  // step leaves most of the memory bandwidth idle, so the CTAs ask the L2 for it while they work (at most 48 MiB).
  const void* prefetch;
  int64_t prefetch_bytes;
  int cos_rows;           // rows of cos_cache / sin_cache; the rotary position is clamped to it (0 = not checked)
} ortb200_gqa_decode_args;
int ortb200_gqa_decode(const ortb200_gqa_decode_args* args, ortb200_stream_t stream);
int64_t ortb200_gqa_decode_workspace_bytes(int B, int N, int H);

// Multi-token attention (prompt / chunked prefill, and encoder self-attention): flash-attention forward on
// tcgen05 with S = Q K^T and O = P V accumulated in tensor memory.
// q / out are [B, S, N, H] described by explicit strides; k / v are addressed as (batch, kv head, position, dim)
// with explicit element strides, so both a [B, Nk, Smax, H] cache and a [B, S, Nk, H] activation work.
// Query token s of batch b sits at absolute position past(b) + s, past(b) = first_prompt ? 0 : seqlens_k[b] + 1 - S,
// and sees keys j < seqlens_k[b] + 1 with (causal ? j <= position : true) and (window > 0 ? j > position - window : true).
// H must be 64 or 128; all strides multiples of 8 elements.
typedef struct {
  const void* q;
  const void* k;
  const void* v;
  const int* seqlens_k;    // [B]; null = every sequence has kv_len keys
  const void* head_sink;   // optional [N]
  void* out;
  int B, S, N, Nk, H;
  int kv_len;              // extent of the position axis of k / v
  int64_t q_strides[3];    // elements: batch, token, head
  int64_t o_strides[3];
  int64_t kv_strides[3];   // elements: batch, head, position
  int first_prompt;
  int causal;
  int window;
  float scale;             // 0 = 1/sqrt(H)
  float softcap;
  int dtype;
  int* status;
  const int* key_mask;     // optional [B, kv_len] int32, 0 = this key is padding for every query of the batch entry
} ortb200_attn_prefill_args;
int ortb200_attn_prefill(const ortb200_attn_prefill_args* args, ortb200_stream_t stream);

// ---------------------------------------------------------------------------
// Small utility kernels.
// rows of `table` [vocab, hidden] selected by int64 ids -> out [n, hidden]
int ortb200_gather_rows(const void* table, const int64_t* ids, void* out, int64_t n, int64_t vocab, int hidden,
                        int elem_bytes, ortb200_stream_t stream);
// argmax over the last dimension: x [rows, n] -> out int64 [rows] (first maximum wins).  `workspace` holds
// ortb200_argmax_workspace_bytes(rows) bytes, zero before the first launch; the kernel leaves it zero.
int ortb200_argmax(const void* x, int64_t* out, int64_t rows, int64_t n, int dtype, void* workspace,
                   int64_t workspace_bytes, ortb200_stream_t stream);
int64_t ortb200_argmax_workspace_bytes(int64_t rows);
// y = act(x + bias[col]) elementwise; bias optional, cols = last dimension
int ortb200_bias_act(const void* x, const void* bias, void* y, int64_t rows, int cols, int act, float alpha, int dtype,
                     ortb200_stream_t stream);
// y = silu(gate) * up for x = [rows, 2 * cols] split in halves (gate | up)
int ortb200_swiglu(const void* x, void* y, int64_t rows, int cols, int dtype, ortb200_stream_t stream);
// standalone rotary embedding on [B, S, N, H] (in -> out, may alias)
int ortb200_rotary(const void* x, void* y, const int64_t* position_ids, int64_t position_offset, const void* cos_cache,
                   const void* sin_cache, int B, int S, int N, int H, int rot_dim, int interleaved, int bnsh, int dtype,
                   ortb200_stream_t stream);

// ---------------------------------------------------------------------------
// Mixture of experts.  ortb200_moe_route runs: softmax + top-k routing (one warp per token), the per-expert histogram,
// the tile plan of the grouped GEMM, and the permutation of the tokens into expert order.  Only the experts
// [expert_begin, expert_end) are served (expert parallelism: the others belong to other ranks and get row_of = -1).
// Afterwards:  ortb200_gemm_grouped(xp -> h), ortb200_gemm_grouped(h -> y), ortb200_moe_combine(y -> out).
typedef struct {
  const void* logits;   // [tokens, E], dtype
  const void* x;        // [tokens, H], 16-bit dtype (bf16 / fp16)
  int tokens, E, k, H;
  int normalize;        // divide the k chosen probabilities by their sum
  int expert_begin, expert_end;
  int tile_rows, max_tiles;   // from ortb200_moe_tile_rows / ortb200_moe_max_tiles
  int dtype;            // of logits
  int* topk_idx;        // out [tokens, k]
  float* topk_w;        // out [tokens, k]
  int* counts;          // scratch [E_local]
  int* offsets;         // out [E_local + 1]
  int* cursors;         // scratch [E_local]
  void* tile_info;      // out int4 [max_tiles]
  int* num_tiles;       // out scalar
  void* xp;             // out [tokens * k, H] rows in expert order (rows of other ranks' experts stay unwritten)
  int* row_of;          // out [tokens, k]: row of (token, choice) in xp, or -1
} ortb200_moe_route_args;
int ortb200_moe_route(const ortb200_moe_route_args* args, ortb200_stream_t stream);
int ortb200_moe_tile_rows(int64_t rows, int experts);
int ortb200_moe_max_tiles(int64_t rows, int experts, int tile_rows);
// out[t] = sum_j topk_w[t, j] * (y[row_of[t, j]] + bias[topk_idx[t, j] - expert_begin]); rows with row_of < 0 are skipped.
int ortb200_moe_combine(const void* y, const void* bias, void* out, int tokens, int H, int k, int expert_begin,
                        const int* topk_idx, const float* topk_w, const int* row_of, int dtype, ortb200_stream_t stream);

// ---------------------------------------------------------------------------
// Collectives as one kernel over the symmetric workspace (same workspace and peer table as the fused GEMM; this
// file's kernels use its upper half).  All ranks must issue the same sequence of calls.
//   ALLREDUCE: out = sum over ranks of in; row_bytes = bytes of the whole tensor (rows ignored).
//   ALLGATHER: in is [rows, row_bytes]; out is [rows, world, row_bytes] (gathering along any axis is this with
//              rows = product of the leading dimensions).
//   ALLTOALL:  in is [world, row_bytes]; out[s] = chunk `rank` of rank s's input.
// Sizes are multiples of 16 bytes, pointers 16-byte aligned; ortb200_symm_collective_max_bytes gives the largest
// message (per-rank input bytes) the workspace can take - larger ones go through the library collective.
enum { ORTB200_COLL_ALLREDUCE = 0, ORTB200_COLL_ALLGATHER = 1, ORTB200_COLL_ALLTOALL = 2 };
typedef struct {
  int op;
  const void* in;
  void* out;
  int64_t rows;
  int64_t row_bytes;
  int dtype;       // all-reduce only
  int world, rank;
  void* peers[8];
  int64_t symm_bytes;
  int* status;
  int use_pdl;
  void* mc_ptr;    // all-reduce: NVLS multicast address of the workspace, or null (peer loads and stores only)
} ortb200_symm_collective_args;
int ortb200_symm_collective(const ortb200_symm_collective_args* args, ortb200_stream_t stream);
int64_t ortb200_symm_collective_max_bytes(int op, int world, int64_t symm_bytes);

// Expert-parallel MoE, last step, as one kernel over the symmetric workspace (same layout and epoch word as
// ortb200_symm_collective): out[t] = sum over the token's top-k experts of topk_w * (expert output + bias), where every
// rank holds only the outputs of its own experts (row_of < 0 elsewhere).  Each rank pushes one pre-summed row per token
// to the token's owner rank, the owner adds them in top-k order and stores the finished row into every rank's copy,
// so all ranks end with the full [T, H] result.  Experts are dealt to ranks in equal blocks of E_local.
typedef struct {
  const void* y;          // [rows, H] outputs of this rank's experts (permuted order)
  const void* bias;       // optional [E_local, H]
  void* out;              // [T, H]
  const int* topk_idx;    // [T, k] global expert ids (identical on every rank)
  const float* topk_w;    // [T, k]
  const int* row_of;      // [T, k] row of y, -1 when the expert is not local
  int T, H, k, E_local, expert_begin;
  int dtype;              // F16 or BF16
  int world, rank;
  void* peers[8];
  int64_t symm_bytes;
  int* status;
  int use_pdl;
} ortb200_moe_combine_symm_args;
int ortb200_moe_combine_symm(const ortb200_moe_combine_symm_args* args, ortb200_stream_t stream);
int64_t ortb200_moe_combine_symm_max_tokens(int world, int k, int H, int64_t symm_bytes);

// Re-arranges MatMulNBits 4-bit weights for the in-kernel expansion: within every 32-bit word (8 weights, low nibble
// = even k) weight 2i moves to bits [4i, 4i+4) and weight 2i+1 to bits [16+4i, 16+4i+4).  B and out are N * K / 2
// bytes; they may not alias.
int ortb200_nbits_prepack(const void* B, void* out, int64_t bytes, ortb200_stream_t stream);

// MatMulNBits weights -> dense rows.  B uint8 [N, n_blocks, block_size * bits / 8] (low nibble = even k), scales
// [N, n_blocks], zero_points packed uint8 [N, ceil(n_blocks * bits / 8)] (zp_is_packed = 1) or typed [N, n_blocks]
// (zp_is_packed = 0) or null (2^(bits-1)); out [N, ldo] with out[n, k] = (q - zp) * scale.  bits = 4 or 8,
// block_size a power of two >= 16, ldo a multiple of 8.
int ortb200_nbits_dequant(const void* B, const void* scales, const void* zero_points, int zp_is_packed, void* out,
                          int64_t N, int K, int bits, int block_size, int64_t ldo, int dtype, ortb200_stream_t stream);

#ifdef __cplusplus
}
#endif
