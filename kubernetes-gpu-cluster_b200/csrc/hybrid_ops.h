// Launchers of the kernels that layer-list ("hybrid") models add to the library: a shape-agnostic linear layer with
// grouped / gathered rows, fp32-residual norms, biased chunk-masked paged attention (soft cap, sink logits), rotary
// positions with a whole-projection norm, the gated linear recurrence (RG-LRU), the matrix memory (mLSTM), the
// mixture-of-experts router, the hyper-connected residual (several streams), the WKV recurrence (also run as gated linear
// attention), the row-wise parts of attention through latents, sliding windows with kept first tokens or pooled blocks,
// short causal convolutions with a state, per-head norms with rotary positions in halves and rotated values, and grouped
// RMS norms before and after a sublayer.  Every mechanism takes its sizes and constants
// as arguments.  `elt` names the storage type of activations and weights: KGE_ELT_BF16 or KGE_ELT_F32; what the
// mechanisms compute in 32 bits (softmax, norms, routers, residual sums, recurrent state and everything that enters a
// recurrence besides projections and short convolutions) is 32-bit in both.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace kge {

enum { KGE_ELT_BF16 = 0, KGE_ELT_F32 = 1 };
enum { ACT_NONE = 0, ACT_GELU_ERF = 1, ACT_GELU_TANH = 2, ACT_SILU = 3, ACT_SIGMOID = 4, ACT_TANH = 5, ACT_RELU2 = 6 };

inline size_t elt_size(int elt) { return elt == KGE_ELT_F32 ? 4 : 2; }

// y[yr(r), n] (+)= alpha * act(scale_r * sum_k x[xr(r), k] * w[n, k] + bias[n])        (w2 == null)
// y[yr(r), n] (+)= alpha * silu(scale_r * x.w[n]) * (scale_r * x.w2[n])                  (w2 != null: gated pair)
//   glu == GLU_CLAMPED_SIGMOID: with g = min(scale_r * x.w[n], glu_limit), u = clamp(scale_r * x.w2[n], -glu_limit,
//   glu_limit) the pair gives alpha * g * sigmoid(glu_alpha * g) * (u + 1)
// Rows r run over [0, T), or - with group_off - over [group_off[z], group_off[z+1]) for each z < nz, where slice z
// reads x at column offset z * x_zs, weights at w + z * w_zs (elements), bias at z * b_zs and writes y at column offset
// z * y_zs.  xrows / yrows (null = identity) gather the input row and scatter the output row; row_scale (null = 1) is
// indexed by r.  Sums run over k in ascending order in fp32, whatever else is in the launch.
struct LinearArgs {
  const void* x = nullptr; int ldx = 0;
  const void* w = nullptr; const void* w2 = nullptr; const void* bias = nullptr;
  void* y = nullptr; int ldy = 0;
  int T = 0, N = 0, K = 0;
  int nz = 1; int64_t x_zs = 0, w_zs = 0, b_zs = 0, y_zs = 0;
  const int32_t* group_off = nullptr;     // device [nz + 1]
  int max_rows = 0;                        // with group_off: an upper bound of any group's row count (0 = T)
  const int32_t* xrows = nullptr; const int32_t* yrows = nullptr;
  const float* row_scale = nullptr;
  int act = ACT_NONE; float alpha = 1.f; bool accumulate = false;
  int glu = 0; float glu_alpha = 1.702f, glu_limit = 0.f;      // gated pairs: GLU_SILU_MUL or GLU_CLAMPED_SIGMOID
  int elt = KGE_ELT_BF16; bool out_f32 = false;
};
enum { GLU_SILU_MUL = 0, GLU_CLAMPED_SIGMOID = 1 };
int linear_any(const LinearArgs& a, cudaStream_t st);

// res[t, :] = float(table[ids[t], :])
int embed_f32(float* res, const int32_t* ids, const void* table, int T, int d, int elt, cudaStream_t st);
// y[r, :] = out_scale * x[rows ? rows[r] : r, :] / sqrt(mean(x^2) + eps) * (offset + w), x fp32, y in elt
int rmsnorm_f32in(void* y, const float* x, const int32_t* rows, const void* w, int R, int d, float eps, float offset, float out_scale, int elt,
                  cudaStream_t st);
// the same rows through a layer norm with a weight and no bias: (x - mean) / sqrt(mean((x - mean)^2) + eps) * w, two passes in fp32
int layernorm_f32in(void* y, const float* x, const int32_t* rows, const void* w, int R, int d, float eps, float out_scale, int elt, cudaStream_t st);
// res[t, :] += sum_i scale[i] * rscale_i(t) * src[i][t, :]   (up to 4 sources in elt, each [T, d] with its own leading
// dimension; rscale_i(t) = rscale[i][t * rs_stride[i]] where a per-row fp32 factor is given, else 1)
struct CombineArgs {
  const void* src[4] = {nullptr, nullptr, nullptr, nullptr}; int ld[4] = {0, 0, 0, 0}; float scale[4] = {0, 0, 0, 0};
  const float* rscale[4] = {nullptr, nullptr, nullptr, nullptr}; int rs_stride[4] = {0, 0, 0, 0};
  int n = 0;
};
int residual_combine(float* res, const CombineArgs& a, int T, int d, int elt, cudaStream_t st);
// RMS norm in groups: the row is cut into `groups` equal consecutive parts, each divided by its own
// sqrt(mean(part^2) + eps); the whole is multiplied by w (as it is) and out_scale.  x fp32, y in elt.
int group_rmsnorm_f32in(void* y, const float* x, const int32_t* rows, const void* w, int R, int d, int groups, float eps, float out_scale, int elt,
                        cudaStream_t st);
// A sublayer's result joins the residual stream through a norm of its own, and the next sublayer's input is formed in the same pass:
//   y[t, :]   = src_scale * sum_i (inner_w[i] ? src_i[t, :] / sqrt(mean(src_i[t, :]^2) + eps) * inner_w[i] : src_i[t, :])      (nsrc <= 2)
//   res[t, :] += gn(y[t, :]) * post_w           gn: the group norm above
//   next_y[t, :] = gn(res[t, :]) * next_w       (next_w != null; next_y in elt)
// Sources and weights in elt, statistics and sums in fp32.
struct PostNormArgs {
  float* res = nullptr;
  const void* src[2] = {nullptr, nullptr}; int ld[2] = {0, 0}; const void* inner_w[2] = {nullptr, nullptr}; int nsrc = 1; float src_scale = 1.f;
  const void* post_w = nullptr; const void* next_w = nullptr; void* next_y = nullptr;
  int T = 0, d = 0, groups = 1; float eps = 1e-5f; int elt = KGE_ELT_BF16;
};
int postnorm_residual(const PostNormArgs& a, cudaStream_t st);
// Causal convolution over time on `C` neighbouring columns of x (row stride ldx), written to y (row stride ldy):
//   y_t[c] = sum_j w[c, j] * x_(t - taps + 1 + j)[c],   w [C, taps], zeros before position 0;
// inputs before a request's first row of this step come from its state slot, which holds the last taps - 1 input rows
// (fp32 [taps - 1, C], oldest first) and is brought up to date at the end.  Sums in fp32, ascending j.
struct ShortConvArgs {
  const void* x = nullptr; int ldx = 0; void* y = nullptr; int ldy = 0; const void* w = nullptr; int C = 0, taps = 1;
  float* state = nullptr; int64_t slot_stride = 0;
  const int32_t* slots = nullptr; const int32_t* qsl = nullptr; const int32_t* positions = nullptr; const int32_t* token_req = nullptr;
  int B = 0, T = 0; int elt = KGE_ELT_BF16;
};
int short_conv_state(const ShortConvArgs& a, cudaStream_t st);
inline int64_t short_conv_state_floats(int C, int taps) { return (int64_t)C * (taps - 1); }
// y[t, n] = silu(gu[t, n]) * gu[t, f + n], n < f (gu [T, 2 f] in elt, the activation in fp32, one rounding)
int silu_mul_halves(void* y, const void* gu, int T, int f, int elt, cudaStream_t st);

// fp32 [R, V] -> 16-bit logits for the samplers (ld_out >= V)
int logits_to_elt16(void* out, const float* in, int R, int V, int ld_out, bool f16, cudaStream_t st);
int elt16_to_f32(float* out, const void* in_bf16, int64_t n, cudaStream_t st);
// soft cap of logits rows, v <- cap * tanh(v / cap) in fp32: on fp32 rows [R, V] in place (l32), and / or on 16-bit rows
// (l16, row stride ld16) in place; with both given the 16-bit rows are read and the capped value goes to both
int softcap_rows(float* l32, void* l16, int R, int V, int ld16, float cap, cudaStream_t st);

// Paged attention with a per-head linear distance bias and an optional chunk mask.
//   score(i, j) = cap(scale * q_i . k_j) - slope_h * (i - j),  slope_h = 2^(-bias_span * (h + 1) / H)   (bias_span = 0: no bias),
//   cap(s) = softcap * tanh(s / softcap) (softcap = 0: s).  With `sinks` (fp32 [H]) the softmax denominator of head h
//   also holds exp(sinks[h]): a logit without key or value, neither scaled nor capped.
//   j visible to i iff j <= i and (chunk == 0 or floor(i / chunk) == floor(j / chunk)), positions counted from the
//   start of the sequence.  With window > 0 only j > i - window is visible that way, and beside those keys either
//   (keep_first > 0) the positions j < keep_first that have left the window, with their own keys and values, or
//   (pool > 0) entry b of the pooled caches for every b < floor((i - window + 1) / pool): one key / value per block of
//   `pool` positions that lies wholly before the window (pool_kv_write makes them).  All of a row's keys share one
//   softmax; the distance bias is not defined for kept or pooled keys (bias_span must be 0 with a window).
//   Softmax in fp32.  q rows are read from a packed projection buffer (row stride ldq elements,
//   head h at column h * dim); K cache [num_blocks, G, block_size, dim], V cache [num_blocks, G, block_size, vdim].
//   out [T, H * vdim] (row stride ldo), multiplied by out_scale.
struct AttnBiasArgs {
  const void* q = nullptr; int ldq = 0; void* out = nullptr; int ldo = 0;
  const void* k_cache = nullptr; const void* v_cache = nullptr;
  const int32_t* block_table = nullptr; int max_blocks = 0;
  const int32_t* seq_lens = nullptr; const int32_t* qsl = nullptr; const int32_t* positions = nullptr;
  const int32_t* token_req = nullptr;      // [T] request index of every token row
  int B = 0, T = 0, H = 0, G = 0, dim = 0, vdim = 0, block_size = 0, chunk = 0;
  int max_q = 0;                           // the longest request's rows in this step (0 = unknown: the per-row kernel runs)
  int num_decode = 0;                      // leading requests that bring one token each: their keys are split over a CTA's warps,
                                           // while requests with many rows give each warp 16 rows of a shared key tile
  float scale = 1.f, bias_span = 0.f, out_scale = 1.f, softcap = 0.f;
  const float* sinks = nullptr;
  int window = 0, keep_first = 0, pool = 0;
  const void* pk_cache = nullptr; const void* pv_cache = nullptr;     // pooled caches [num_blocks, G, pool_slots, dim / vdim]
  int pool_slots = 0;                      // pooled entries per page: entry b of a request lives in its page b / pool_slots
  int elt = KGE_ELT_BF16;
};
int attn_bias_chunk(const AttnBiasArgs& a, cudaStream_t st);
inline int pool_slots_per_block(int block_size, int pool) { return (block_size + pool - 1) / pool; }
// Pooled keys and values: for every token of the step whose position p ends a block of `pool` positions
// ((p + 1) % pool == 0), entry b = p / pool of the pooled caches <- the mean (fp32, positions in ascending order, one
// rounding to the storage type) of the `pool` cached keys / values of positions b * pool .. p, read through the block
// table.  Runs after the step's keys and values are in the caches.
struct PoolKvArgs {
  const void* k_cache = nullptr; const void* v_cache = nullptr; void* pk_cache = nullptr; void* pv_cache = nullptr;
  const int32_t* block_table = nullptr; int max_blocks = 0; const int32_t* positions = nullptr; const int32_t* token_req = nullptr;
  int T = 0, G = 0, dim = 0, vdim = 0, block_size = 0, pool = 1, pool_slots = 1;
  int elt = KGE_ELT_BF16;
};
int pool_kv_write(const PoolKvArgs& a, cudaStream_t st);
// k / v rows of a packed projection buffer -> paged caches (slot = block * block_size + offset, < 0 skips)
int kv_write_any(const void* k, int ldk, const void* v, int ldv, const int64_t* slots, void* k_cache, void* v_cache, int T, int G,
                 int dim, int vdim, int block_size, int elt, cudaStream_t st);

// Rotary positions for packed q / k projections, with what comes before and after them in one pass over a token's row:
//   - optional RMS norm over the WHOLE q projection (all heads at once; weight q_norm_w [H * dim]) and over the whole
//     k projection (k_norm_w [G * dim]), in fp32: x / sqrt(mean(x^2) + eps) * w;
//   - rotation of the first rot_dims dimensions of every head in interleaved pairs (2i, 2i + 1):
//     (u, v) -> mult * (u cos a - v sin a, v cos a + u sin a), a = position * freq[i]; the angle is formed and reduced
//     in double precision, freq [rot_dims / 2] comes from rotary_frequencies();
//   - q is written back in place, the rotated k goes to the paged key cache, and the value cache receives either the
//     rows of `v` or (v == null) the key projection as it came in, before norm and rotation.
// Caches as in kv_write_any: [num_blocks, G, block_size, dim]; slot < 0 skips the cache writes.
struct RotaryArgs {
  void* q = nullptr; int ldq = 0; const void* k = nullptr; int ldk = 0; const void* v = nullptr; int ldv = 0;
  const void* q_norm_w = nullptr; const void* k_norm_w = nullptr; float eps = 1e-5f;
  const double* freq = nullptr; float mult = 1.f; int rot_dims = 0;
  const int32_t* positions = nullptr; const int64_t* slots = nullptr;
  void* k_cache = nullptr; void* v_cache = nullptr;
  int T = 0, H = 0, G = 0, dim = 0, vdim = 0, block_size = 0;
  int elt = KGE_ELT_BF16;
};
int rotary_norm_kvwrite(const RotaryArgs& a, cudaStream_t st);
// The same pass with norms per head and pairs in halves.  q [T, H * dim] and k [T, G * dim] are RMS-normed per head
// (norm_q / norm_k; the weight of `dim` numbers is shared by all heads, null = no weight), then the first rot_dims
// dimensions of every head turn in pairs (i, i + rot_dims / 2) by position * freq[i]; q is written back in place, k goes
// to the key cache.  v [T, G * vdim] goes to the value cache as it is, or (v_freq != null) with ALL vdim dimensions turned
// in pairs (m, m + vdim / 2) by position * v_freq[m].  Norm statistics, angles (double precision) and rotation in fp32.
struct HeadRotaryArgs {
  void* q = nullptr; int ldq = 0; const void* k = nullptr; int ldk = 0; const void* v = nullptr; int ldv = 0;
  bool norm_q = false, norm_k = false; const void* q_norm_w = nullptr; const void* k_norm_w = nullptr; float eps = 1e-5f;
  const double* freq = nullptr; int rot_dims = 0; const double* v_freq = nullptr;
  const int32_t* positions = nullptr; const int64_t* slots = nullptr;
  void* k_cache = nullptr; void* v_cache = nullptr;
  int T = 0, H = 0, G = 0, dim = 0, vdim = 0, block_size = 0;
  int elt = KGE_ELT_BF16;
};
int head_norm_rotary_kvwrite(const HeadRotaryArgs& a, cudaStream_t st);
// x[t, h, :n] (row stride ldx, head h at column h * n) turns in pairs (m, m + n / 2) by sign * position[t] * freq[m], in place
int rotate_heads_halves(void* x, int ldx, const int32_t* positions, const double* freq, int T, int H, int n, float sign, int elt, cudaStream_t st);

// freq[i] = base^(-2i / dims), i < dims / 2; with YaRN scaling (factor > 0): ramp_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1)
// between lo = max(floor(c(fast)), 0) and hi = min(ceil(c(slow)), dims - 1), c(t) = dims * ln(original / (2 pi t)) / (2 ln base);
// freq_i <- freq_i / factor * ramp_i + freq_i * (1 - ramp_i) and *mult = 0.1 ln(factor) + 1 (else 1).  Host only.
void rotary_frequencies(int dims, double base, double factor, double original, double fast, double slow, double* freq, float* mult);

// Gated linear recurrence (RG-LRU).  yx [T, 2 * width]: the y branch's pre-activation, then the x branch (biases in).
//   u = causal per-channel conv of x (taps weights per channel, last tap on the current token; inputs before position 0
//       are zero; inputs before this step's first token come from the slot's conv tail)
//   r = sigmoid(gate_r), i = sigmoid(gate_i): pre-activations of block-diagonal projections of u, given in fp32
//   a = exp(-decay_c * r * softplus(lam));  S <- a S + sqrt(1 - a^2) * i * u;  out = S * gelu_tanh(y)
// State per slot: S [width] and the last taps - 1 inputs of the conv, all fp32; a request whose first row is position 0
// starts from zero.  rglru_conv writes u (elt); rglru_scan runs the recurrence and writes out (elt) and the state.
struct RglruArgs {
  const void* yx = nullptr; void* u = nullptr; const float* gates = nullptr;   // gates [T, 2 * width]: r then i
  void* out = nullptr;
  const void* conv_w = nullptr; const void* conv_b = nullptr; const void* lam = nullptr;
  float* state = nullptr; int64_t slot_stride = 0;     // floats between slots; this layer's state starts at `state`
  const int32_t* slots = nullptr; const int32_t* qsl = nullptr; const int32_t* positions = nullptr; const int32_t* token_req = nullptr;
  int B = 0, T = 0, width = 0, taps = 1;
  float decay_c = 8.f;
  int elt = KGE_ELT_BF16;
};
int rglru_conv(const RglruArgs& a, cudaStream_t st);
int rglru_scan(const RglruArgs& a, cudaStream_t st);
inline int64_t rglru_state_floats(int width, int taps) { return (int64_t)width * taps; }   // S + (taps - 1) conv inputs

// Matrix memory (mLSTM) with a running maximum m that starts at 0.
//   i~ = cap * tanh(i_pre / cap), f~ = logsigmoid(cap * tanh(f_pre / cap))   (gate pre-activations in fp32, [T, 2 * H]: i then f)
//   m' = max(f~ + m, i~);  S <- exp(f~ + m - m') S + exp(i~ - m') k v^T;  n likewise with k;  q scaled by q_scale
//   o = S^T q / (max(|n . q|, exp(-m')) + den_eps), divided by its root mean square over vdim (eps), times norm_w,
//   times sigmoid(gate) -> out [T, H * vdim], multiplied by out_scale.
// State per slot and head: S [dim, vdim], n [dim], m, all fp32.
struct MlstmArgs {
  const void* q = nullptr; const void* k = nullptr; const void* v = nullptr; const void* g = nullptr; int ld = 0;   // one packed buffer
  const float* gates = nullptr;
  const void* norm_w = nullptr; void* out = nullptr; int ldo = 0;
  float* o_scratch = nullptr;              // fp32 [T, H * vdim]: with it (and dim <= 128) the value columns of a head are split
                                           // over several blocks with the state in registers, and a second kernel normalises
  float* state = nullptr; int64_t slot_stride = 0;
  const int32_t* slots = nullptr; const int32_t* qsl = nullptr; const int32_t* positions = nullptr;
  int B = 0, T = 0, H = 0, dim = 0, vdim = 0;
  float cap = 1.f, q_scale = 1.f, eps = 1e-5f, den_eps = 1e-6f, out_scale = 1.f;
  int elt = KGE_ELT_BF16;
};
int mlstm_step(const MlstmArgs& a, cudaStream_t st);
inline int64_t mlstm_state_floats(int H, int dim, int vdim) { return (int64_t)H * ((int64_t)dim * vdim + dim + 1); }

// Mixture-of-experts routing: logits z = W_router h (+ b_router) in fp32, scores sigmoid(z) (score_fn 0) or softmax(z) (1),
// the `top` largest chosen (ties to the lower index), weights = scores * weight_scale, renormalised to sum 1 first if renorm; score_fn 2:
// the `top` largest LOGITS are chosen and the weights are the softmax over the chosen logits only.  Produces for every
// expert the list of (token, choice) pairs routed to it: group_off [E + 1], perm_token [T * top] (the token row of
// every permuted row), perm_weight [T * top], perm_dest [T * top] (row t * top + choice of the output buffer).
struct MoeRouteArgs {
  const void* h = nullptr; int ldh = 0; const void* w_router = nullptr; const void* b_router = nullptr;
  const void* w_extra = nullptr; float* extra_sigmoid = nullptr;      // one more row [d]: extra_sigmoid[t] = sigmoid(w_extra . h_t) (a per-token gate)
  int T = 0, d = 0, E = 0, top = 1, score_fn = 0; bool renorm = false; float weight_scale = 1.f;
  int32_t* group_off = nullptr; int32_t* perm_token = nullptr; float* perm_weight = nullptr; int32_t* perm_dest = nullptr;
  int32_t* choice_expert = nullptr; float* choice_weight = nullptr;     // scratch [T * top] each
  // pad > 1: every expert's rows start at a multiple of `pad` (group_off holds the padded offsets; perm_* have rows_padded
  // entries, -1 in perm_token / perm_dest marks a row without a pair), and tile_group [rows_padded / pad] names the expert
  // of every tile of `pad` rows - what the grouped tensor-core GEMM reads
  int pad = 0, rows_padded = 0; int32_t* tile_group = nullptr;
  int elt = KGE_ELT_BF16;
};
int moe_route(const MoeRouteArgs& a, cudaStream_t st);
// routed rows made contiguous per expert: xperm[p, :] = bf16(perm_weight[p] * h[perm_token[p], :]) (null weights: 1); and back: out[perm_dest[p], :] = operm[p, :]
int moe_gather_rows(void* xperm, const void* h, int ldh, const int32_t* perm_token, const float* perm_weight, int np, int d, cudaStream_t st);
int moe_scatter_rows(void* out, const void* operm, const int32_t* perm_dest, int np, int d, cudaStream_t st);

// Hyper-connected residual: S copies ("streams") of the fp32 residual stream, xs [T, S, d].
//   embed_norm_streams: every stream of token t <- float(table[ids[t]]) (norm_w == null) or its RMS norm times norm_w
//   stream_norm:        u = sum_s in_w[s] xs[row, s, :] (in_w null: plain sum);  y[r, :] = out_scale * u / sqrt(mean(u^2) + eps) * w
//                       (row = rows ? rows[r] : r; y in elt); sum_out (fp32 [R, d], optional) receives u
//   stream_combine:     with y[t, :] = y32[t, :] + sum_i scale_i * rscale_i(t) * src_i[t, :] (the sources of CombineArgs, summed
//                       in order; y32 optional) and z = mult * col_scale[:] * y (col_scale null: 1), all streams at once from
//                       the old ones: xs[t, j, :] <- sum_s mix[s * S + j] xs[t, s, :] + out_w[j] * z   (mix null: identity; out_w null: 1)
// in_w / out_w / mix / col_scale are fp32 on the device.  S <= 8.
int embed_norm_streams(float* xs, const int32_t* ids, const void* table, const void* norm_w, int T, int d, int S, float eps, int elt, cudaStream_t st);
struct StreamNormArgs {
  void* y = nullptr; const float* xs = nullptr; const float* in_w = nullptr; const int32_t* rows = nullptr; const void* w = nullptr;
  float* sum_out = nullptr;
  int R = 0, d = 0, S = 1; float eps = 1e-5f, out_scale = 1.f; int elt = KGE_ELT_BF16;
};
int stream_norm(const StreamNormArgs& a, cudaStream_t st);
struct StreamCombineArgs {
  float* xs = nullptr; CombineArgs src; const float* y32 = nullptr;
  const float* col_scale = nullptr; const float* mix = nullptr; const float* out_w = nullptr;
  float mult = 1.f; int T = 0, d = 0, S = 1; int elt = KGE_ELT_BF16;
  // the next sublayer's read in the same pass (next_y != null): next_y[t, :] = n(sum_j next_in[j] * new xs[t, j, :]) * next_w
  const float* next_in = nullptr; const void* next_w = nullptr; void* next_y = nullptr; float eps = 1e-5f;
};
int stream_combine(const StreamCombineArgs& a, cudaStream_t st);

// WKV: a matrix-valued linear recurrence per head with a per-token, per-key-channel decay and a bonus for the current token.
//   wkv_shift_mix: with h' the previous token's row of h (zeros at position 0; the slot's saved row where the step
//     starts inside a sequence), mixes[z, t, :] = h + (h' - h) * mu[z, :] for z < nmix (mixes [nmix, T, d] in elt, mu
//     [nmix, d] in elt); afterwards the slot keeps the last row of every request of the step (fp32).
//   wkv_scan: per head, o_t = (S + diag(u) k_t v_t^T)^T r_t, then S <- diag(w_t) S + k_t v_t^T with
//     w_t = exp(-exp(decay_pre_t)) (decay_pre fp32 [T, H * dim], the logit with its bias in); S [dim, dim] fp32 per slot and
//     head, zero at position 0.  o is divided by its root mean square over the head (eps), multiplied by norm_w and by
//     silu(gate_pre) and written to out [T, H * dim] (elt).  u fp32 [H * dim].  o32: fp32 scratch [T, H * dim].
struct WkvArgs {
  const void* h = nullptr; int ldh = 0; const void* mu = nullptr; void* mixes = nullptr; int nmix = 5; int d = 0;
  const void* r = nullptr; const void* k = nullptr; const void* v = nullptr; const void* gate_pre = nullptr; int ld = 0;
  const float* decay_pre = nullptr; const float* u = nullptr; const void* norm_w = nullptr;
  float* o32 = nullptr; void* out = nullptr; int ldo = 0;
  float* state = nullptr; int64_t slot_stride = 0;     // this layer's part of slot 0: [d] saved row, then [H, dim, dim]
  const int32_t* slots = nullptr; const int32_t* qsl = nullptr; const int32_t* positions = nullptr; const int32_t* token_req = nullptr;
  int B = 0, T = 0, H = 0, dim = 0;
  int max_q = 0;                           // the longest request's rows in this step (0 = unknown: token by token)
  float eps = 1e-5f;
  // gated linear attention on the same kernels: value size vdim (0 = dim; S is [dim, vdim], v / gate_pre / out / o32 /
  // norm_w rows are H * vdim wide), decay_mode 1: w_t = sigmoid(decay_pre_t)^(1 / tau) = exp(logsigmoid(decay_pre_t) / tau),
  // read_after: o_t = S_t^T r_t with S_t the state AFTER the update (no bonus u), r multiplied by r_scale in fp32
  int vdim = 0, decay_mode = 0; bool read_after = false; float tau = 1.f, r_scale = 1.f;
  int elt = KGE_ELT_BF16;
};
int wkv_shift_mix(const WkvArgs& a, cudaStream_t st);
int wkv_scan(const WkvArgs& a, cudaStream_t st);
inline int64_t wkv_state_floats(int d, int H, int dim) { return (int64_t)d + (int64_t)H * dim * dim; }
inline int64_t gla_state_floats(int H, int dim, int vdim) { return (int64_t)H * dim * vdim; }     // WkvArgs with d = 0

// Attention through latents, the parts around the attention kernel.
//   segment_rmsnorm: up to two column ranges of the rows of x (elt, row stride ldx) are RMS-normed in fp32 and written
//     packed: out_i[t, :] = x[t, col_i : col_i + n_i] / sqrt(mean(.^2) + eps) * w_i.
//   latent_rotary_kvwrite: q [T, H * dim] in place: the last rot_part dimensions of every head are the rotated part, of
//     which the first rot_dims turn in interleaved pairs by position * freq[i] (angle in double precision); the shared
//     key part k_rot [T, rot_part] turns the same way; head h's key cache row is [k_nope[t, h * (dim - rot_part) ...] | turned
//     k_rot], its value cache row v[t, h * vdim ...].  Caches as in kv_write_any with G = H.
//   sigmoid_gate_mul: y[t, c] <- y[t, c] * sigmoid(g[t, c]), c < n.
struct SegNormArgs {
  const void* x = nullptr; int ldx = 0; int T = 0; float eps = 1e-5f; int elt = KGE_ELT_BF16;
  int nseg = 1; int col[2] = {0, 0}; int n[2] = {0, 0}; const void* w[2] = {nullptr, nullptr}; void* out[2] = {nullptr, nullptr}; int ldo[2] = {0, 0};
};
int segment_rmsnorm(const SegNormArgs& a, cudaStream_t st);
struct LatentKvArgs {
  void* q = nullptr; int ldq = 0; const void* k_nope = nullptr; int ldk = 0; const void* v = nullptr; int ldv = 0; const void* k_rot = nullptr; int ldr = 0;
  const double* freq = nullptr; int rot_dims = 0, rot_part = 0;
  const int32_t* positions = nullptr; const int64_t* slots = nullptr;
  void* k_cache = nullptr; void* v_cache = nullptr;
  int T = 0, H = 0, dim = 0, vdim = 0, block_size = 0;
  int elt = KGE_ELT_BF16;
  bool vec = false;                        // set by the launcher: every part is a whole number of 16-byte pieces
};
int latent_rotary_kvwrite(const LatentKvArgs& a, cudaStream_t st);
int sigmoid_gate_mul(void* y, int ldy, const void* g, int ldg, int T, int n, int elt, cudaStream_t st);

}  // namespace kge
