// Host launchers of the kernels behind the non-Llama model designs: a shape-agnostic linear layer (plain, batched per
// head, or grouped per expert), Dynamic-Tanh norm fused with the fp32 residual update, a hashed bigram embedding,
// gated linear attention (decayed outer-product state per sequence slot; per-channel learned decays or one constant per
// head), latent attention (paged low-rank KV with a shared rotated key and a sliding window), softmax attention over
// paged keys and values with grouped heads, a sliding window and kept first tokens, hyper-connections (several residual
// streams read and written through small mixing weights) with RMS norm, expert routing (softmax or sigmoid scores,
// optionally group-limited, or a softmax over the chosen logits), the matrix-memory recurrence with exponential gating
// (mLSTM), a sinusoidal position embedding, a residual step with a norm on both sides of the sublayer, a short causal
// convolution over time with its carried inputs, the selective scan of Mamba, chunked visibility and a softmax sink for
// the paged attention, a learned position embedding, two normed branches summed, and the gated activations they use.
//
// Storage type: every activation / weight matrix is either bf16 or fp32 (DType); the residual stream, recurrent
// states, router scores, decays, softmax and norm statistics are always fp32.  All pointers are device pointers.
// Launchers return 0 on success and a negative number on a bad shape or a launch error.
#pragma once
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

namespace b200 {

enum DType { DT_BF16 = 0, DT_F32 = 1 };
inline size_t dtype_bytes(DType t) { return t == DT_BF16 ? 2 : 4; }

// ---------------------------------------------------------------- linear (linear.cu)
enum LinearAct { LIN_NONE = 0, LIN_RELU2 = 1 };   // epilogue on the fp32 accumulator: identity, max(y, 0)^2
// Y[b][t, n] = act( sum_k X[b][row(t), k] * W[b'][n, k] ),  t < T, n < N.
//   batch > 1: X, W, Y advance by xbs / wbs / ybs elements per batch index (per-head projections inside wider rows).
//   x_rows (optional): row(t) = x_rows[t], a negative entry reads a zero row and its output row is not written.
//   tile_group (optional, needs T % 64 == 0 capacity): rows [64 i, 64 i + 64) use weight matrix W + tile_group[i] * wbs;
//     a negative entry skips the tile (expert-grouped rows padded to the tile size).
//   row_scale (optional, fp32): the accumulator of row t is multiplied by row_scale[t] before act, which is the product
//     of the scaled input row, (s x) W^T = s (x W^T), without a scaled copy of x.
//   bias (optional, fp32 [N]): added to the (scaled) accumulator before act.
// The accumulation order of one output element never depends on T or on the other rows (k ascending inside a tile
// kernel, a fixed lane pattern in the few-row kernel), so a row's result does not depend on what shares the batch.
struct LinearArgs {
  const void* X; const void* W; void* Y;
  DType tx, tw, ty;
  int T, N, K;
  int ldx, ldw, ldy;
  int batch; long long xbs, wbs, ybs;
  const int* x_rows;
  const int* tile_group;
  int act;
  const float* row_scale;
  const float* bias;
};
inline LinearArgs linear_args(const void* X, DType tx, const void* W, DType tw, void* Y, DType ty, int T, int N, int K) {
  LinearArgs a = {X, W, Y, tx, tw, ty, T, N, K, K, K, N, 1, 0, 0, 0, nullptr, nullptr, LIN_NONE, nullptr, nullptr};
  return a;
}
int linear(const LinearArgs& a, cudaStream_t st);
// `rows` rows (a handful: the expert choices of a decode step), row r reading X row src_rows[r] (or r / src_div), writing Y row
// dst_rows[r], with weight matrix W + groups[r] * wbs (row_scale[r] applies); a.T, a.batch, x_rows and tile_group are not used.
// group_limit > 0: a row whose group is negative or >= group_limit has no weight matrix and is skipped (its output row is
// not written): the choices of a router that are not matrices at all, such as identity experts.
struct PickedRows {
  int rows;
  const int* src_rows; int src_div;
  const int* dst_rows;
  const int* groups;
  int group_limit = 0;
};
int linear_picked_rows(const LinearArgs& a, const PickedRows& p, cudaStream_t st);

// ---------------------------------------------------------------- embedding, norm, activations (norm_act.cu)
// x[t] = embed[ids[t]] + bigram[row], row = (prev * mul_prev + id * mul_cur) mod buckets, or row `buckets` when
// prev_ids[t] < 0 (the first token of a sequence).  x is fp32 [T, W]; tables are [*, W] of type tw.
int embed_bigram(const void* embed, const void* bigram, DType tw, const int* ids, const int* prev_ids, float* x, int T, int W,
                 int vocab, int buckets, long long mul_prev, long long mul_cur, cudaStream_t st);
// Dynamic Tanh with the residual update in front of it.  For r < rows, t = row_index ? row_index[r] : r:
//   if (a || f) x[t] += mult * (a[t] + f[t])   (fp32, in place; a, f of type ta, either may be null)
//   if (y)      y[r] = tanh(alpha[0] * x[t]) * w + b          (w, b, alpha fp32; y of type ty)
int residual_dyt(float* x, const void* a, const void* f, DType ta, float mult, const float* w, const float* b, const float* alpha,
                 void* y, DType ty, const int* row_index, int rows, int W, cudaStream_t st);
// Clamped gated unit: row t of gu (leading dimension ldgu) holds gate [F] | up [F]; g = min(gate, limit), u = clamp(up, -limit, limit),
// y = g * sigmoid(slope * g) * (u + up_offset).  limit = INFINITY, slope = 1, up_offset = 0 is the plain SiLU-gated unit.
int glu_clamped(const void* gu, int ldgu, void* y, int ldy, DType t, int T, int F, float limit, float slope, cudaStream_t st,
                float up_offset = 1.0f);
// y[t, i] = act(y[t, i] + bias[i]) in place, i < n (leading dimension ldy; bias fp32, may be null; act: LinearAct)
int bias_act(void* y, int ldy, const float* bias, int act, DType t, int T, int n, cudaStream_t st);
// y[t, i] *= sigmoid(g[t, i]), i < n (leading dimensions ldy, ldg)
int sigmoid_gate(void* y, int ldy, const void* g, int ldg, DType t, int T, int n, cudaStream_t st);
// p[i] = offset + scale * u_i, u uniform in [-1, 1) from a counter hash of (seed, i): seeded random weights for benchmarks
int fill_uniform(void* p, DType t, size_t n, uint64_t seed, float scale, float offset, cudaStream_t st);
int argmax_f32(const float* logits, int* out, int S, int V, cudaStream_t st);

// ---------------------------------------------------------------- gated linear attention (gla.cu)
// Per sequence and head: S <- diag(alpha_t) S + k_t v_t^T, o_t = S^T (q_t * q_scale), alpha = sigmoid(z + z_bias)^(inv_tau),
// all in fp32.  q, k, v are column blocks of one row-major buffer (leading dimension ld, column offsets q_off / k_off /
// v_off; heads x dim, heads x dim, heads x vdim).  z: fp32 [T, heads * dim] pre-activations, replaced by the decays.  states: fp32 [slot][heads][dim][vdim].
// seqs: int [nseq][8] = {first row, rows, first position, state slot, ...}; a sequence whose first position is 0 starts
// from a zero state whatever its slot held.  o: fp32 [T, heads * vdim].
// head_decay (optional, fp32 [heads]): every key channel of head h decays by the constant head_decay[h] (the scalar-decay
// linear attention, S <- lambda_h S + k v^T); z and z_bias are then unused and may be null.  act: GLA_ACT_SILU applies
// x * sigmoid(x) to q, k and v as they are read (q before q_scale).
// tok_decay with tok_kscale (fp32 [T, heads]): every channel of head h decays by tok_decay[t, h] at token t and the key is
// multiplied by tok_kscale[t, h] as it is read, S <- d_t S + (s_t k_t) v_t^T (scalar gates that change from token to
// token); z, z_bias and head_decay are then unused.  With them, nstate (fp32 [slot][heads][dim]) and nq (fp32 [T, heads])
// make the scan carry the running key sum n_t = d_t n_(t-1) + s_t k_t beside the state and write nq[t, h] = n_t . (q_t *
// q_scale), which normalised recurrences divide by.
// rope (optional, [position][rot_dims / 2] of (cos, sin)): the first rot_dims dimensions of every query and key head are
// rotated by the token's position as they are read, dimension i paired with i + rot_dims / 2 (the rotate-half layout), in
// fp32; k_scale multiplies the key after the rotation.
enum GlaAct { GLA_ACT_NONE = 0, GLA_ACT_SILU = 1 };
struct GlaArgs {
  const void* qkv; DType t; int ld, q_off, k_off, v_off;
  float* z; const float* z_bias; float inv_tau, q_scale;   // z is overwritten with the decays
  int T;                                                      // rows of z (tokens in the step)
  float* states; const int* seqs; int nseq;
  int heads, dim, vdim;
  float* o;
  const float* head_decay = nullptr;
  int act = GLA_ACT_NONE;
  const float* tok_decay = nullptr; const float* tok_kscale = nullptr;
  float* nstate = nullptr; float* nq = nullptr;
  const float2* rope = nullptr; int rot_dims = 0; float k_scale = 1.f;
};
int gla_scan(const GlaArgs& a, cudaStream_t st);
// y[t, h * vdim + :] (leading dimension ldy) = o[t, h, :] / sqrt(mean(o^2) + eps) * w * silu(g[t, h, :])   (w: fp32 [vdim], shared by the heads)
int gla_out_gate(const float* o, const void* g, int ldg, const float* w, float eps, void* y, int ldy, DType t, int T, int heads, int vdim,
                 cudaStream_t st);
// The general form: the unit-RMS norm runs per head over vdim with w [vdim] shared by the heads (joint = false) or once
// over the token's concatenated heads with w [heads * vdim] (joint = true); the gate is silu(g) or sigmoid(g); the result
// is multiplied by out_scale before it is rounded to the storage type.
enum GateAct { GATE_SILU = 0, GATE_SIGMOID = 1 };
// Per-head form only: w_full = true reads the weight as [heads * vdim] (every head its own) instead of [vdim]; with den_nq
// and den_floor (fp32 [T, heads]) the outputs of head h are divided by max(|den_nq[t, h]|, den_floor[t, h]) + den_eps
// before the norm (a normalised recurrence: den_nq is the product n . q of its running key sum with the query).
// w may be null: a norm without a weight.
struct OutGateArgs {
  const float* o; const void* g; int ldg; const float* w; float eps;
  void* y; int ldy; DType t;
  int T, heads, vdim;
  bool joint; int gate_act; float out_scale;
  bool w_full = false;
  const float* den_nq = nullptr; const float* den_floor = nullptr; float den_eps = 0.f;
};
int recurrent_out_gate(const OutGateArgs& a, cudaStream_t st);
// The scalar gates of the matrix-memory recurrence with exponential gating (mLSTM), per token and head, in fp32:
//   log input gate  i = cap * tanh(zi / cap),   log forget gate  f = logsigmoid(cap * tanh(zf / cap))   (cap <= 0: no cap)
//   running log-scale  m_t = max(f_t + m_(t-1), i_t),  m before the first token of a sequence is 0
//   keep[t, h] = exp(f + m_(t-1) - m_t),  take[t, h] = exp(i - m_t),  floor[t, h] = exp(-m_t)
// so that the stored state is the true one divided by exp(m): S_t = keep S_(t-1) + take k v^T (gla_scan with tok_decay =
// keep, tok_kscale = take).  pre: fp32 [T, ld] pre-activations with bias, zi of head h at column h, zf at heads + h.
// mstate: fp32 [slot][heads], read when the sequence's first position is above 0, written at the end of the step.
struct MlstmGateArgs {
  const float* pre; int ld; float cap;
  float* keep; float* take; float* floor;
  float* mstate; const int* seqs; int nseq; int heads;
};
int mlstm_gates(const MlstmGateArgs& a, cudaStream_t st);

// ---------------------------------------------------------------- latent attention (latent_attention.cu)
// Rotation table for interleaved pairs (2i, 2i+1): cs[p][i] = (cos, sin)(p * base^(-2i/dims)), computed in double.
int rope_table_interleaved(float2* table, int max_pos, int dims, double base, cudaStream_t st);
// Per token: the first kv_rank columns of dkv are unit-RMS-normed (eps inside the root) and scaled by norm_w -> cache row,
// the next rot_dim columns are rotated (first rot_dims of them) -> cache row tail; the rotated part of every query head
// (q laid out [heads][dim + rot_dim]) is rotated into qlat[t][h][kv_rank ...] (fp32, row stride heads * (kv_rank + rot_dim)).
// cache: [slot][kv_rank + rot_dim] of type t, slot = page * page_size + offset as given by slots[t].
struct LatentPrepArgs {
  const void* q; int ldq; const void* dkv; int lddkv; DType t;
  const float* norm_w; float eps;
  const float2* rope; int rot_dims;
  const int* positions; const int* slots;
  void* cache; float* qlat;
  int T, heads, dim, rot_dim, kv_rank;
};
int latent_prep(const LatentPrepArgs& a, cudaStream_t st);
// Sliding-window softmax attention in latent space: for token t at position p of sequence s, keys j with
// max(0, p - window + 1) <= j <= p; score = qlat[t, h] . cache[j] * scale; olat[t, h] = sum_j softmax_j * cache[j][:kv_rank].
struct LatentAttnArgs {
  const float* qlat; const void* cache; DType t;
  const int* positions; const int* seq_of_tok; const int* block_tables; int max_blocks, page;
  float* olat;
  int T, heads, kv_rank, rot_dim, window; float scale;
  const int* seqs; int nseq;   // the step's per-sequence table ({first row, rows, first position, ...}); needed by the tensor-core kernel
  int max_ctx;                 // longest context (position of a last token + 1) in the step, for the split decision
  float* split_ws; long long split_ws_floats;   // optional workspace of the split form: [rows][splits][kv_rank + 2] fp32
};
int latent_attention(const LatentAttnArgs& a, cudaStream_t st);

// ---------------------------------------------------------------- softmax attention, windowed with kept first tokens (window_attention.cu)
// Rotation table for interleaved pairs with YaRN-style frequency scaling: f_i = base^(-2i/dims) is blended towards
// f_i / factor by a ramp between the pair indices at which `fast` and `slow` rotations fit into `original` positions,
// and cos and sin are multiplied by 0.1 ln(factor) + 1.  yarn == nullptr gives the plain table.  Computed in double.
struct RopeYarn { double factor, original, fast, slow; };
int rope_table_yarn(float2* table, int max_pos, int dims, double base, const RopeYarn* yarn, cudaStream_t st);
// Per token: the first rot_dims dimensions of every query head (heads x dim at q) and key head (kv_heads x dim at k) are
// rotated by the token's position (pairs (2i, 2i+1)), then each head is divided by its root mean square over dim (eps
// inside the root; unit_norm = false skips that).  Queries go to qn (fp32 [T, heads * dim]); keys and values
// (kv_heads x vdim at v) go to the token's cache row: cache [slot][kv_heads * dim | kv_heads * vdim] of type t.
// q_norm_w / k_norm_w (optional, fp32 [dim], shared by the heads) multiply the normed query / key.  q_gain_every > 0
// multiplies the query at position p by 1 + q_gain_coef * ln(floor((p + 1) / q_gain_every) + 1).  v_blend (optional, type
// t, [T, kv_heads * vdim] with leading dimension ld_blend): the cached value is (1 - v_lambda) v + v_lambda v_blend (the
// same token's values of an earlier layer); v_raw_out (optional, same shape, leading dimension ld_raw) receives v as it
// came in, for later layers to blend with.  rot_dims = 0 needs no table.
struct QkPrepArgs {
  const void* q; const void* k; const void* v; int ld; DType t;   // column blocks of one row-major buffer
  const float2* rope; int rot_dims;
  bool unit_norm; float eps;
  const int* positions; const int* slots;
  float* qn; void* cache;
  int T, heads, kv_heads, dim, vdim;
  const float* q_norm_w = nullptr; const float* k_norm_w = nullptr;
  float q_gain_coef = 0.f; int q_gain_every = 0;
  const void* v_blend = nullptr; int ld_blend = 0; float v_lambda = 0.f;
  void* v_raw_out = nullptr; int ld_raw = 0;
};
int qk_rope_norm_cache(const QkPrepArgs& a, cudaStream_t st);
// The preparation of an attention whose queries and keys pass a short causal convolution over time and whose values are
// the convolved keys.  qk: [T, heads * dim | kv_heads * dim], neighbouring columns of one row-major buffer (the
// projections).  Per token, in fp32: every channel is convolved with its taps (conv_w [channels, taps], the last tap is
// the token's own; the taps - 1 inputs before a portion's first token come from conv_state [slot][taps - 1][channels],
// zeros before the sequence's start; conv_w null: no convolution); the convolved keys are the values of the cache row;
// the whole query row (all heads at once) and the whole key row are divided by their root mean square (eps inside the
// root) and multiplied by q_norm_w [heads * dim] / k_norm_w [kv_heads * dim]; the first rot_dims dimensions of every head
// are rotated by the token's position, dimension i paired with i + rot_dims / 2 (rotate-half layout; rope as
// rope_table_yarn writes it); query head h is multiplied by q_head_scale[h] (optional: a temperature per head).
// Queries go to qn (fp32 [T, heads * dim]), keys to the cache row [kv_heads * dim (keys) | kv_heads * dim (values)].
// The carried inputs are written afterwards by short_conv_carry over the same columns.
struct ConvQkPrepArgs {
  const void* qk; int ld; DType t;
  const float* conv_w; int taps; const float* conv_state;
  const float* q_norm_w; const float* k_norm_w; float eps;
  const float2* rope; int rot_dims;
  const float* q_head_scale;
  const int* positions; const int* slots; const int* seq_of_tok; const int* seqs;
  float* qn; void* cache;
  int T, heads, kv_heads, dim;
};
int conv_qk_prep(const ConvQkPrepArgs& a, cudaStream_t st);
// Softmax attention of token t (position p of its sequence) over the cached keys j <= p with p - j < window or
// j < keep_first (kept tokens stay at their own positions).  Query head h reads key/value head h / (heads / kv_heads).
// score = qn . k * scale, softmax in fp32.  y[t, h * vdim + :] = out_scale * o * sigmoid(gate[t, h * vdim + :]) (gate of
// type t with leading dimension ldg, may be null: no gate), rounded once to type t (leading dimension ldy).
// softcap > 0: score <- softcap * tanh(score / softcap) after the scale.  gate_per_head: the gate holds one number per
// (token, head), gate[t * ldg + h], instead of one per output column.
// chunk > 0 replaces the sliding window by chunked visibility: the token at position p sees the keys j <= p of its own
// chunk, floor(j / chunk) = floor(p / chunk), chunks counted from position 0 of the sequence (window is then unused;
// keep_first still applies).  sink (optional, fp32 [heads]): the softmax denominator of head h gets the extra term
// exp(sink[h]), which belongs to no cached token, adds nothing to the numerator and stays outside scale and cap.
struct WindowAttnArgs {
  const float* qn; const void* cache; DType t;
  const int* positions; const int* seq_of_tok; const int* block_tables; int max_blocks, page;
  const void* gate; int ldg; float out_scale;
  void* y; int ldy;
  int T, heads, kv_heads, dim, vdim, window, keep_first; float scale;
  const int* seqs; int nseq; int max_ctx;
  float softcap = 0.f; bool gate_per_head = false;
  int chunk = 0; const float* sink = nullptr;
};
int window_attention(const WindowAttnArgs& a, cudaStream_t st);

// ---------------------------------------------------------------- short causal convolution, selective scan (ssm.cu)
// y[t, c] = act(bias[c] + sum_j w[c, j] * u[t - taps + 1 + j, c]) over the tokens of t's own sequence: the last tap is the
// token's own input, inputs before a portion's first token come from state [slot][taps - 1][C] (fp32, oldest first) when
// the portion starts past position 0, and are zeros before the sequence's start.  u: C columns of a row-major buffer of
// type t (leading dimension ldu); w fp32 [C, taps]; bias fp32 [C] or null; y of type ty.  Computed in fp32.
// short_conv_carry writes the state a step leaves behind (the last taps - 1 inputs of every sequence, older ones shifted
// in from the old state when the portion is shorter); it runs after every kernel of the step that reads the old state.
enum ConvAct { CONV_NONE = 0, CONV_SILU = 1 };
struct ShortConvArgs {
  const void* u; int ldu; DType t;
  const float* w; const float* bias; int act;
  void* y; int ldy; DType ty;
  float* state;
  const int* seq_of_tok; const int* seqs; int nseq;
  int T, C, taps;
};
int short_conv(const ShortConvArgs& a, cudaStream_t st);
int short_conv_carry(const ShortConvArgs& a, cudaStream_t st);
// The selective scan of Mamba, per sequence, channel c and state index n, in fp32:
//   d = softplus(dt[t, c]);  S[c, n] <- exp(d * A[c, n]) * S[c, n] + d * x[t, c] * B[t, n];
//   y[t, c] = (sum_n S[c, n] * C[t, n] + D[c] * x[t, c]) * silu(z[t, c])
// x, z: [T, inner] column blocks of type t (x after its convolution and activation, z the gate's pre-activation); dt: fp32
// [T, inner] pre-activations of the step size (with their bias); bc: fp32 rows holding B at column b_off and C at c_off
// ([state] each); A fp32 [inner, state] (negative); D fp32 [inner]; states fp32 [slot][inner][state], zero for a
// sequence whose first position is 0 whatever its slot held.  Sequential in the token: the same operations in the same
// order however a prompt is cut.
struct SelectiveScanArgs {
  const void* x; int ldx; const void* z; int ldz; DType t;
  const float* dt; int lddt;
  const float* bc; int ldbc, b_off, c_off;
  const float* A; const float* D;
  float* states; const int* seqs; int nseq;
  void* y; int ldy;
  int inner, state;
};
int selective_scan(const SelectiveScanArgs& a, cudaStream_t st);

// ---------------------------------------------------------------- hyper-connections, RMS norm (hyper.cu)
// x[s][t] = embed[ids[t]] * scale for every stream s (fp32; stream s starts at x + s * stream_stride).
int embed_scaled(const void* embed, DType tw, const int* ids, float* x, int T, int W, int vocab, float scale, int streams,
                 long long stream_stride, cudaStream_t st);
// One boundary between two sublayers on `streams` fp32 residual streams (1..8).  For r < rows, t = row_index ? row_index[r] : r:
//   if (y)  all streams at once from the old ones: x_j[t] <- sum_s mix[s * streams + j] * x_s[t] + out[j] * y[t]
//           (mix null: identity; out null: ones; with one stream and both null this is the plain residual sum)
//   u = sum_s in[s] * x_s[t]                                   (in null: the plain sum of the streams)
//   if (h)  h[r] = norm_w ? u / sqrt(mean(u^2) + eps) * norm_w : u      (fp32 statistics; h of type th)
struct HyperArgs {
  float* x; int streams; long long stream_stride;
  const void* y; DType ty;
  const float* mix; const float* out; const float* in;
  const float* norm_w; float eps;
  void* h; DType th;
  const int* row_index; int rows; int W;
  // gated write-back (optional): y[t, i] is multiplied by sigmoid(gate[t * ldg + i] + gate_bias[i]) before it enters the
  // streams (gate of type tg, pre-activations of a projection; gate_bias fp32, may be null)
  const void* gate = nullptr; DType tg = DT_BF16; int ldg = 0; const float* gate_bias = nullptr;
};
int hyper_step(const HyperArgs& a, cudaStream_t st);
// x[s][t] = embed[ids[t]] + pos_table[pos[t]] for every stream s (fp32): a learned position vector, not scaled.
// pos_table: [max_pos, W] of type tw; a position at or past max_pos reads the last row.
int embed_learned_pos(const void* embed, const void* pos_table, DType tw, const int* ids, const int* pos, float* x, int T, int W, int vocab,
                      int max_pos, int streams, long long stream_stride, cudaStream_t st);
// Two branches, each RMS-normed over the width with its own weight, summed: for t < T
//   y[t] = scale * (a[t] / sqrt(mean(a[t]^2) + eps) * wa + b[t] / sqrt(mean(b[t]^2) + eps) * wb)
// a, b: [T, W] of type t; wa, wb fp32 [W]; y of type ty; fp32 statistics, one rounding.
struct BranchNormArgs {
  const void* a; const void* b; DType t;
  const float* wa; const float* wb; float eps, scale;
  void* y; DType ty;
  int T, W;
};
int branch_norm_sum(const BranchNormArgs& a, cudaStream_t st);

// Sinusoidal positions added to the embedding: x[t] = embed[ids[t]] + s(pos[t]), where column c of s(p) belongs to the
// pair i = c / 2 with angle p * base^(-2i/W) and carries its sine (c even) or cosine (c odd).  freq: [(W + 1) / 2] float2,
// the double-precision frequency of every pair split into two floats (sinusoid_freq_table), so that the angle p * f keeps
// its low bits at large positions; x is fp32 [T, W].
int sinusoid_freq_table(float2* freq, int W, double base, cudaStream_t st);
int embed_sinusoid(const void* embed, DType tw, const int* ids, const int* pos, const float2* freq, float* x, int T, int W, int vocab,
                   cudaStream_t st);
// One boundary between two sublayers of a design with a norm on both sides of every sublayer, on one fp32 residual.
// For r < rows, t = row_index ? row_index[r] : r:
//   if (y)  u = y[t] + y_bias;  x[t] <- x[t] + (post_w ? u / sqrt(mean(u^2) + eps) * post_w : u)      (y_bias fp32, may be null)
//   if (h)  h[r] = pre_w ? x[t] / sqrt(mean(x[t]^2) + eps) * pre_w : x[t]                             (fp32 statistics; h of type th)
// post_w and pre_w are the multiplicative weights themselves (a stored offset from one is added at load).
struct SandwichArgs {
  float* x;
  const void* y; DType ty; const float* y_bias;
  const float* post_w; const float* pre_w; float eps;
  void* h; DType th;
  const int* row_index; int rows; int W;
};
int sandwich_step(const SandwichArgs& a, cudaStream_t st);

// ---------------------------------------------------------------- mixture of experts (moe.cu)
// scores: fp32 [T, E] router logits in, clobbered.  softmax over E; experts form `groups` equal groups of neighbours, a
// group's score is its largest member, only the `keep` best groups are eligible; the `top` largest eligible scores are
// chosen (ties: lower index) and used unchanged as weights.  topk_ids / topk_w: [T, top].
// score_fn: MOE_SOFTMAX as above, MOE_SIGMOID scores every expert by sigmoid(z) on its own (no normalisation over E),
// MOE_TOP_SOFTMAX ranks the experts by the logits themselves and weights the chosen ones by the softmax over the chosen
// logits only.
enum MoeScore { MOE_SOFTMAX = 0, MOE_SIGMOID = 1, MOE_TOP_SOFTMAX = 2 };
// ld: leading dimension of scores (0: E); columns past E are left alone (a design may keep other fp32 outputs there).
// select_bias (optional, fp32 [E]; MOE_SOFTMAX and MOE_SIGMOID): experts (and groups) are ranked by score + select_bias,
// the weights stay the scores themselves.
int moe_route(float* scores, int* topk_ids, float* topk_w, int T, int E, int groups, int keep, int top, cudaStream_t st,
              int score_fn = MOE_SOFTMAX, int ld = 0, const float* select_bias = nullptr);
// Sort the T * top (token, choice) pairs by expert into 64-row tiles: sorted_rows[cap] = token of each sorted row or -1,
// tile_group[cap / 64] = expert of each tile or -1, pair_pos[T * top] = sorted row of each pair.  cap >= T*top + E*64.
// expert_rows (optional): [E][2] = {first sorted row, rows} of every expert.
// topk_w with sorted_w (optional): sorted_w[cap] = the router weight of each sorted row (0 for padding), for designs that
// scale an expert's input instead of its output.
// matrices (0: E): experts at or above it have no weights (identity experts); their tiles are marked -1, so that the
// grouped launches skip them, while their rows keep their places in the order.
int moe_align(const int* topk_ids, int T, int top, int E, int* sorted_rows, int* tile_group, int* pair_pos, int cap, cudaStream_t st,
              int* expert_rows = nullptr, const float* topk_w = nullptr, float* sorted_w = nullptr, int matrices = 0);
// out[t] = sum_k topk_w[t, k] * y[pair_pos[t * top + k]]   (y [cap, W] fp32 or bf16, k ascending)
int moe_combine(const void* y, DType ty, const int* pair_pos, const float* topk_w, void* out, DType t, int T, int top, int W, cudaStream_t st);
// out[t] = sum_k w[t, k] * y[pair_pos[t * top + k]] + sigmoid(add_gate[t * ld_gate]) * add[t]: the routed experts plus a
// shared expert behind a per-token gate.  topk_w may be null (every weight 1: the weight was applied to the expert's
// input); add ([T, W]) is of type t and may be null (no shared expert); add_gate is fp32 and may be null (gate 1).
int moe_combine_add(const void* y, DType ty, const int* pair_pos, const float* topk_w, const void* add, const float* add_gate, int ld_gate,
                    void* out, DType t, int T, int top, int W, cudaStream_t st);
// The same with identity experts: a choice topk_ids[t, k] >= matrices contributes w[t, k] * x[t] (the expert's input row
// itself, x of type t) instead of a row of y, which is not read for it.
int moe_combine_identity(const void* y, DType ty, const int* pair_pos, const float* topk_w, const int* topk_ids, int matrices, const void* x,
                         void* out, DType t, int T, int top, int W, cudaStream_t st);
// bf16 helpers of the per-expert tensor-core path: x rows in sorted order (negative source row -> zeros; with row_scale the
// row is multiplied by row_scale[r] in fp32 and rounded once), max(p, 0)^2 in place
int moe_gather_bf16(const void* x, const int* sorted_rows, void* out, int rows, int W, cudaStream_t st, const float* row_scale = nullptr);
int relu2_bf16(void* p, long long n, cudaStream_t st);

}  // namespace b200
