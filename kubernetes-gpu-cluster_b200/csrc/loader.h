// HF-layout model directory reader: config.json -> ModelSpec, *.safetensors -> host tensors
// (mmap, zero-copy), converted to bf16 on demand.  Host only.
#pragma once
#include <stdint.h>

#include <map>
#include <string>
#include <vector>

namespace kge {

// One layer of a layer-list ("hybrid") model: which token mixer it has, that mixer's sizes and constants, and its
// feed-forward.  Every number comes from config.json; the kernels take them as parameters.
struct HybridLayerSpec {
  enum Mixer { RGLRU = 0, PARALLEL = 1, ATTENTION = 2, WKV = 3, LATENT = 4, WINDOW_GLA = 5, POOLED = 6 };
  enum Mlp { NONE = 0, DENSE = 1, MOE = 2 };
  int mixer = RGLRU;
  // gated linear recurrence (RG-LRU): two branches of `width`, gates block-diagonal in `blocks` parts, causal conv of `conv` taps
  int width = 0, blocks = 1, conv = 1;
  // attention side of a parallel mixer: H query heads on G key/value heads, key size `dim`, value size `vdim`, a linear
  // distance bias per head, visibility limited to the query's own chunk of `chunk` positions (0 = whole causal prefix)
  int heads = 0, kv_heads = 0, dim = 0, vdim = 0, chunk = 0;
  float scale = 1.f, left_scale = 1.f;
  // matrix-memory side (mLSTM): heads x (dim x vdim) state, gate pre-activations soft-capped at gate_cap
  int m_heads = 0, m_dim = 0, m_vdim = 0;
  float gate_cap = 0.f, right_scale = 1.f;
  // attention alone (ATTENTION; heads / kv_heads / dim / vdim / scale as above): scores soft-capped at `softcap` (0 = not),
  // a learned per-head sink logit in the softmax denominator, RMS norm of the whole q and k projections (before they are
  // split into heads), values taken from the key projection as it leaves the matrix product (no value matrix), rotary
  // positions on the first rot_dims dimensions of every head in interleaved pairs, with YaRN frequency scaling
  // (yarn_factor 0 = plain frequencies)
  float softcap = 0.f;
  bool sink = false, qk_norm = false, v_from_k = false;
  int rot_dims = 0;
  double rot_base = 10000.0, yarn_factor = 0.0, yarn_original = 0.0, yarn_fast = 32.0, yarn_slow = 1.0;
  // matrix-valued linear recurrence with a per-channel, per-token decay (WKV): `heads` x (`dim` x `dim`) state, every
  // projection reads its own blend of the token and the one before it, the decay's logit comes through a low-rank pair
  // of `decay_rank` columns (taken from the checkpoint's shapes when 0)
  int decay_rank = 0;
  // attention through latents (LATENT): keys and values are up-projections of one normed latent of `kv_rank` numbers per
  // token; a key is [dim - rot_part unrotated | rot_part rotated] where the rotated part comes straight from the
  // down-projection and is shared by all heads; queries come through a normed latent of `q_rank` numbers (0: one
  // matrix); rotary positions act on the first rot_dims of the rot_part; out_gate: the heads' outputs are multiplied by
  // sigmoid(W_g h) before the output matrix.  heads = kv_heads, dim counts the whole key, vdim the value.
  int q_rank = 0, kv_rank = 0, rot_part = 0;
  bool out_gate = false;
  // windowed attention beside gated linear attention (WINDOW_GLA), both reading the same row; each side's output is
  // RMS-normed over the model width with a weight of its own and the mixer's result is half their sum.
  //   attention side (heads / kv_heads / dim / vdim / scale / rot_dims / rot_base as above): q, k and v carry biases and pass a
  //   causal convolution of `conv` taps per channel; q and k are RMS-normed per head with one weight of `dim` numbers
  //   (head_norm); rotary positions act on the first rot_dims dimensions of a head in pairs (i, i + rot_dims / 2)
  //   (rot_halves); the values turn over all vdim dimensions by their own position before they are cached and the head's
  //   output turns back by the query's position (v_rot); position i sees j <= i with i - j < window or j < keep_first.
  //   linear-attention side: m_heads x (m_dim x m_vdim) state, q scaled by m_dim^(-1/2), a decay per key channel
  //   sigmoid(z)^(1 / tau) whose logit z comes through a low-rank pair with a bias, read-out after the update, a per-head
  //   RMS norm (one weight of m_vdim numbers) and a silu gate.
  // windowed attention over pooled blocks (POOLED): q, k, v and the output carry biases; q and k are divided by their
  // root mean square per head (head_norm without a weight); no rotation; position i sees j with 0 <= i - j < window
  // and one key / value - the mean of the cached ones - for every block of `pool` positions that ends at or before i - window.
  int window = 0, keep_first = 0, pool = 0;
  bool head_norm = false, rot_halves = false, v_rot = false;
  float tau = 1.f;
  // feed-forward
  int mlp = NONE;
  int ff = 0;                                    // dense
  float ff_limit = 0.f;                          // dense: > 0 - a clamped gated unit (gate, up, down) with this limit; 0 - up, GELU, down
  bool ff_silu_bias = false;                     // dense: down(silu(gate h + b) * (up h + b)) + b, every projection with a bias
  int experts = 0, top = 0, expert_ff = 0, shared_ff = 0;   // mixture of experts (+ an always-on shared expert if shared_ff > 0)
  // how the experts are chosen and weighed: ROUTE_SIGMOID_IN - sigmoid scores, the weight multiplies the expert's input;
  // ROUTE_SOFTMAX_TOP - the largest logits (router bias added), softmax over the chosen logits only, the weight multiplies
  // the expert's output
  // ROUTE_SOFTMAX_ALL - softmax over all experts, the largest scores chosen, weight = score * router_scale (not
  // renormalised), multiplies the expert's output
  enum Route { ROUTE_SIGMOID_IN = 0, ROUTE_SOFTMAX_TOP = 1, ROUTE_SOFTMAX_ALL = 2 };
  int route = ROUTE_SIGMOID_IN;
  float router_scale = 1.f;
  bool router_bias = false;
  // the experts' gated unit: GLU_SILU - silu(gate) * up; GLU_CLAMPED - g = min(gate, limit), u = clamp(up, -limit, limit),
  // g * sigmoid(1.702 g) * (u + 1)
  // GLU_NONE_RELU2 - no gate: down(relu(up h)^2)
  enum Glu { GLU_SILU = 0, GLU_CLAMPED = 1, GLU_NONE_RELU2 = 2 };
  int glu = GLU_SILU;
  float expert_limit = 0.f, shared_limit = 0.f;
  bool shared_gate = false;                      // the shared expert's output is multiplied by sigmoid(w_sg . h), one number per token
  int weights_of = -1;                           // >= 0: this layer owns no tensors and runs with that layer's (cache and state stay its own)
  int tensor_index = -1;                         // the 'l<i>.' prefix of this layer's tensors (-1: its place in the list)
  bool has_cache() const { return mixer == PARALLEL || mixer == ATTENTION || mixer == LATENT || mixer == WINDOW_GLA || mixer == POOLED; }
};

struct ModelSpec {
  std::string model_type;       // "opt" | "llama" | "qwen2" | "qwen3" | "safupel" | "girolorn" | "zezilix" | "balenex"
  // layer-list models (config.json "architecture"): per-layer descriptions and the multiplier of the logits
  std::vector<HybridLayerSpec> hybrid;
  float logit_scale = 1.f;
  float logit_softcap = 0.f;    // > 0: logits <- cap * tanh(logits / cap)
  // norms of a layer-list model: one RMS norm (weight applied as 1 + w) that mixer and feed-forward both read, or
  // (hyb_prenorm_pair) a norm before the mixer and, after the mixer's sum, another before the feed-forward;
  // hyb_layernorm: mean-centred layer norm with a weight and no bias instead of the RMS norm
  bool hyb_prenorm_pair = false, hyb_layernorm = false;
  // norm_groups > 1: an RMS norm cuts its row into that many equal consecutive parts and divides each by its own root
  // mean square; hyb_postnorm: every sublayer's result goes through a norm of its own (weights norm1b / norm2b) before it
  // is added to the residual stream; norm weights multiply as they are
  int norm_groups = 1;
  bool hyb_postnorm = false;
  // hyper-connected residual: `streams` >= 1 copies of the residual stream, read through per-sublayer input weights,
  // mixed by a streams x streams matrix and written through output weights (0: one plain residual stream); every
  // sublayer's result is multiplied by residual_mult and, element by element, by a per-layer scale vector; the
  // embedding goes through the model's norm before the first layer
  int streams = 0;
  float residual_mult = 1.f;
  bool embed_norm = false;
  bool is_hybrid() const { return !hybrid.empty(); }
  bool qkv_bias = false;        // qwen2: q/k/v projections carry a bias
  bool qk_norm = false;         // qwen3: RMSNorm over head_dim on q and k, per head, before RoPE
  int vocab = 0, d = 0, L = 0, H = 0, KV = 0, hd = 0, ffn = 0, max_pos = 0;
  float eps = 1e-5f;
  bool tied = false;
  double rope_theta = 10000.0;
  double rope_factor = 0.0, rope_low = 1.0, rope_high = 4.0;   // factor 0 => no llama3 scaling
  int rope_orig_max = 8192;
  int bos = -1, eos = -1;
  std::string torch_dtype;      // config.json torch_dtype / dtype ("float16", "bfloat16", "float32", or empty)
  bool is_opt() const { return model_type == "opt"; }
};

struct HostTensor {
  const uint8_t* data = nullptr;   // inside an mmap
  std::string dtype;               // "BF16" | "F16" | "F32" | "I32"
  std::vector<int64_t> shape;
  int64_t numel() const { int64_t n = 1; for (auto s : shape) n *= s; return n; }
};

class ModelDir {
 public:
  ~ModelDir();
  // Reads config.json (required) and maps every *.safetensors file (may be none).
  bool open(const std::string& dir, std::string* err);
  const ModelSpec& spec() const { return spec_; }
  bool has_weights() const { return !tensors_.empty(); }
  const HostTensor* find(const std::string& name) const;
  // Rows [r0, r1) x cols [c0, c1) of a 2-D (or all of a 1-D, r-range only) tensor as bf16 bits.
  bool read_bf16(const std::string& name, int64_t r0, int64_t r1, int64_t c0, int64_t c1,
                 std::vector<uint16_t>* out, std::string* err) const { return read_16(name, r0, r1, c0, c1, false, out, err); }
  // The same slice as bfloat16 bits (f16 = false) or IEEE half bits (f16 = true), converted from whatever the file holds.
  bool read_16(const std::string& name, int64_t r0, int64_t r1, int64_t c0, int64_t c1, bool f16,
               std::vector<uint16_t>* out, std::string* err) const;
  // A whole tensor of any rank as 32-bit floats (BF16 / F16 / F32 widen exactly; I32 tables convert by value).
  bool read_f32(const std::string& name, std::vector<float>* out, std::string* err) const;

 private:
  struct Map { void* base; size_t len; };
  ModelSpec spec_;
  std::map<std::string, HostTensor> tensors_;
  std::vector<Map> maps_;
};

}  // namespace kge
