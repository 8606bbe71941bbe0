#include "loader.h"

#include "half_bits.h"

#include <dirent.h>
#include <fcntl.h>
#include <string.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <algorithm>
#include <fstream>
#include <sstream>

#include "json.h"

namespace kge {

ModelDir::~ModelDir() {
  for (auto& m : maps_) munmap(m.base, m.len);
}

static bool read_file(const std::string& path, std::string* out) {
  std::ifstream f(path, std::ios::binary);
  if (!f) return false;
  std::stringstream ss;
  ss << f.rdbuf();
  *out = ss.str();
  return true;
}

// the feed-forward entry of a layer ('mlp': null for none)
static bool parse_hybrid_mlp(const Json& l, HybridLayerSpec* hp, std::string* err) {
  HybridLayerSpec& h = *hp;
  const Json* f = l.get("mlp");
  if (f && f->is_obj()) {
    const std::string kind = f->str_or("kind", "");
    if (kind == "dense") { h.mlp = HybridLayerSpec::DENSE; h.ff = (int)f->int_or("ff", 0); h.ff_limit = (float)f->num_or("limit", 0.0); if (h.ff <= 0) { *err = "config.json: dense mlp without ff"; return false; } }
    else if (kind == "moe") {
      h.mlp = HybridLayerSpec::MOE;
      const Json *ex = f->get("expert"), *ro = f->get("router"), *sh = f->get("shared");
      if (!ex || !ro) { *err = "config.json: moe mlp needs 'expert' and 'router'"; return false; }
      h.expert_ff = (int)ex->int_or("ff", 0); h.experts = (int)ro->int_or("experts", 0); h.top = (int)ro->int_or("top", 1);
      if (sh && sh->is_obj()) { h.shared_ff = (int)sh->int_or("ff", 0); h.shared_limit = (float)sh->num_or("limit", 0.0); }
      h.expert_limit = (float)ex->num_or("limit", 0.0);
      h.router_scale = (float)ro->num_or("scale", 1.0);
      if (h.expert_ff <= 0 || h.experts <= 0 || h.top <= 0 || h.top > h.experts) { *err = "config.json: bad moe sizes"; return false; }
    } else { *err = "config.json: unknown mlp kind '" + kind + "'"; return false; }
  }
  return true;
}

// Layer-list models: config.json carries "architecture" and a "layers" array instead of HF's flat sizes.
static bool parse_hybrid(const Json& j, ModelSpec* s, std::string* err) {
  s->model_type = "safupel";
  s->vocab = (int)j.int_or("vocab", 0);
  s->d = (int)j.int_or("width", 0);
  s->logit_scale = (float)j.num_or("logit_scale", 1.0);
  if (const Json* n = j.get("norm")) s->eps = (float)n->num_or("eps", 1e-5);
  s->max_pos = 1 << 20;                 // positions enter through computed biases and masks only: no table bounds them
  s->torch_dtype = "bfloat16";
  s->bos = (int)j.int_or("bos_token_id", -1);
  s->eos = (int)j.int_or("eos_token_id", -1);
  const Json* ls = j.get("layers");
  if (!ls || !ls->is_arr() || ls->arr.empty()) { *err = "config.json: 'layers' must be a non-empty array"; return false; }
  for (const Json& l : ls->arr) {
    HybridLayerSpec h;
    const std::string type = l.str_or("type", "");
    const Json* m = l.get("mixer");
    if (!m || !m->is_obj()) { *err = "config.json: a layer has no 'mixer'"; return false; }
    if (type == "rglru") {
      h.mixer = HybridLayerSpec::RGLRU;
      h.width = (int)m->int_or("width", 0); h.blocks = (int)m->int_or("blocks", 1); h.conv = (int)m->int_or("conv", 1);
      if (h.width <= 0 || h.blocks <= 0 || h.width % h.blocks || h.conv < 1 || h.conv > 16) { *err = "config.json: bad rglru sizes"; return false; }
    } else if (type == "parallel") {
      h.mixer = HybridLayerSpec::PARALLEL;
      const Json *a = m->get("left"), *r = m->get("right");
      if (!a || !r) { *err = "config.json: a parallel mixer needs 'left' and 'right'"; return false; }
      h.heads = (int)a->int_or("heads", 0); h.kv_heads = (int)a->int_or("kv_heads", h.heads);
      h.dim = (int)a->int_or("dim", 0); h.vdim = (int)a->int_or("vdim", h.dim);
      h.scale = (float)a->num_or("scale", 1.0);
      if (const Json* mk = a->get("mask")) h.chunk = (int)mk->int_or("size", 0);
      h.m_heads = (int)r->int_or("heads", 0); h.m_dim = (int)r->int_or("dim", 0); h.m_vdim = (int)r->int_or("vdim", h.m_dim);
      h.gate_cap = (float)r->num_or("gate_cap", 0.0);
      h.left_scale = (float)m->num_or("left_scale", 1.0); h.right_scale = (float)m->num_or("right_scale", 1.0);
      if (h.heads <= 0 || h.kv_heads <= 0 || h.heads % h.kv_heads || h.dim <= 0 || h.vdim <= 0 || h.m_heads <= 0 || h.m_dim <= 0 ||
          h.m_vdim <= 0 || h.gate_cap <= 0.f || h.chunk < 0) { *err = "config.json: bad parallel-mixer sizes"; return false; }
    } else { *err = "config.json: unknown layer type '" + type + "' (rglru, parallel)"; return false; }
    if (!parse_hybrid_mlp(l, &h, err)) return false;
    s->hybrid.push_back(h);
  }
  s->L = (int)s->hybrid.size();
  if (s->vocab <= 0 || s->d <= 0) { *err = "config.json misses a required size"; return false; }
  return true;
}

// Girolorn: a layer list of attention mixers (soft-capped scores, a sink logit per head, RMS norm over the whole q / k
// projections, values = the key projection, interleaved partial rotary positions with YaRN scaling) and mixtures of
// experts (softmax over the chosen logits, clamped gated units, a gated shared expert); weight-only layer norms before
// the mixer and before the feed-forward; layers may run with another layer's tensors; soft-capped logits.
static bool parse_girolorn(const Json& j, ModelSpec* s, std::string* err) {
  s->model_type = "girolorn";
  s->vocab = (int)j.int_or("vocab", 0);
  s->d = (int)j.int_or("width", 0);
  s->logit_softcap = (float)j.num_or("logit_softcap", 0.0);
  if (const Json* n = j.get("norm")) s->eps = (float)n->num_or("eps", 1e-5);
  s->hyb_prenorm_pair = s->hyb_layernorm = true;
  s->max_pos = 1 << 20;                 // rotary angles are computed from the position: no table bounds them
  s->torch_dtype = "bfloat16";
  s->bos = (int)j.int_or("bos_token_id", -1);
  s->eos = (int)j.int_or("eos_token_id", -1);
  const Json* ls = j.get("layers");
  if (!ls || !ls->is_arr() || ls->arr.empty()) { *err = "config.json: 'layers' must be a non-empty array"; return false; }
  for (const Json& l : ls->arr) {
    HybridLayerSpec h;
    const std::string type = l.str_or("type", "");
    const Json* m = l.get("mixer");
    if (!m || !m->is_obj()) { *err = "config.json: a layer has no 'mixer'"; return false; }
    if (type != "attention") { *err = "config.json: unknown layer type '" + type + "' (attention)"; return false; }
    h.mixer = HybridLayerSpec::ATTENTION;
    h.heads = (int)m->int_or("heads", 0); h.kv_heads = (int)m->int_or("kv_heads", h.heads);
    h.dim = (int)m->int_or("dim", 0); h.vdim = (int)m->int_or("vdim", h.dim);
    h.scale = (float)m->num_or("scale", 1.0);
    h.softcap = (float)m->num_or("softcap", 0.0);
    h.sink = h.qk_norm = h.v_from_k = true;
    if (const Json* r = m->get("rot")) {
      if (r->is_obj()) {
        h.rot_dims = (int)r->int_or("dims", 0); h.rot_base = r->num_or("base", 10000.0);
        const Json* sc = r->get("scaling");
        if (sc && sc->is_obj()) {
          h.yarn_factor = sc->num_or("factor", 0.0); h.yarn_original = sc->num_or("original", 0.0);
          h.yarn_fast = sc->num_or("fast", 32.0); h.yarn_slow = sc->num_or("slow", 1.0);
          if (h.yarn_factor <= 0.0 || h.yarn_original <= 0.0 || h.yarn_fast <= 0.0 || h.yarn_slow <= 0.0) { *err = "config.json: bad rotary scaling"; return false; }
        }
      }
    }
    if (h.heads <= 0 || h.kv_heads <= 0 || h.heads % h.kv_heads || h.dim <= 0 || h.vdim != h.dim || h.rot_dims < 0 || h.rot_dims > h.dim ||
        h.rot_dims % 2 || h.rot_base <= 0.0 || h.softcap < 0.f) { *err = "config.json: bad attention sizes (values are the keys: vdim = dim)"; return false; }
    if (!parse_hybrid_mlp(l, &h, err)) return false;
    if (h.mlp == HybridLayerSpec::DENSE) { *err = "config.json: this architecture has no dense mlp"; return false; }
    if (h.mlp == HybridLayerSpec::MOE) {
      h.route = HybridLayerSpec::ROUTE_SOFTMAX_TOP; h.router_bias = true; h.glu = HybridLayerSpec::GLU_CLAMPED; h.shared_gate = h.shared_ff > 0;
      if (h.expert_limit <= 0.f || (h.shared_ff > 0 && h.shared_limit <= 0.f)) { *err = "config.json: an expert needs a positive 'limit'"; return false; }
    }
    if (const Json* wo = l.get("weights_of")) {
      if (!wo->is_num()) { *err = "config.json: 'weights_of' must be a layer index"; return false; }
      h.weights_of = (int)wo->as_i64();
      const int self = (int)s->hybrid.size();
      if (h.weights_of < 0 || h.weights_of >= self || s->hybrid[h.weights_of].weights_of >= 0) { *err = "config.json: 'weights_of' must name an earlier layer with tensors of its own"; return false; }
      const HybridLayerSpec& o = s->hybrid[h.weights_of];
      if (o.heads != h.heads || o.kv_heads != h.kv_heads || o.dim != h.dim || o.mlp != h.mlp || o.experts != h.experts || o.expert_ff != h.expert_ff ||
          o.shared_ff != h.shared_ff) { *err = "config.json: a layer with 'weights_of' must have that layer's sizes"; return false; }
    }
    s->hybrid.push_back(h);
  }
  s->L = (int)s->hybrid.size();
  if (s->vocab <= 0 || s->d <= 0) { *err = "config.json misses a required size"; return false; }
  return true;
}

// Zezilix: a layer list of WKV recurrences and latent attention (two kinds: queries through a normed latent, or
// queries from one matrix with a sigmoid output gate), dense clamped gated units or softmax-routed mixtures of ungated
// squared-ReLU experts, on a hyper-connected residual (several streams, per-sublayer read / mix / write weights) with
// a multiplier and a per-layer scale vector on every sublayer's result; the embedding is normed; a run of layers may
// repeat with the same tensors (every pass with a cache and state of its own), which the list below holds unrolled.
static bool parse_zezilix(const Json& j, ModelSpec* s, std::string* err) {
  s->model_type = "zezilix";
  s->vocab = (int)j.int_or("vocab", 0);
  s->d = (int)j.int_or("width", 0);
  if (const Json* n = j.get("norm")) s->eps = (float)n->num_or("eps", 1e-5);
  s->hyb_prenorm_pair = true;
  s->embed_norm = true;
  s->streams = (int)j.int_or("streams", 1);
  s->residual_mult = (float)j.num_or("residual_mult", 1.0);
  s->max_pos = 1 << 20;                 // rotary angles are computed from the position: no table bounds them
  s->torch_dtype = "bfloat16";
  s->bos = (int)j.int_or("bos_token_id", -1);
  s->eos = (int)j.int_or("eos_token_id", -1);
  if (s->streams < 1 || s->streams > 8) { *err = "config.json: 'streams' must be 1 .. 8"; return false; }
  const Json* ls = j.get("layers");
  if (!ls || !ls->is_arr() || ls->arr.empty()) { *err = "config.json: 'layers' must be a non-empty array"; return false; }
  std::vector<HybridLayerSpec> own;
  for (const Json& l : ls->arr) {
    HybridLayerSpec h;
    const std::string type = l.str_or("type", "");
    const Json* m = l.get("mixer");
    if (!m || !m->is_obj()) { *err = "config.json: a layer has no 'mixer'"; return false; }
    h.heads = (int)m->int_or("heads", 0);
    const int dim = (int)m->int_or("dim", 0);
    if (type == "wkv") {
      h.mixer = HybridLayerSpec::WKV;
      h.dim = h.vdim = dim; h.kv_heads = h.heads;
      h.decay_rank = (int)m->int_or("decay_rank", 0);
      if (h.heads <= 0 || dim <= 0 || h.decay_rank < 0) { *err = "config.json: bad wkv sizes"; return false; }
    } else if (type == "latent_attention" || type == "latent_attention_2") {
      h.mixer = HybridLayerSpec::LATENT;
      h.out_gate = type == "latent_attention_2";
      h.kv_heads = h.heads;
      h.rot_part = (int)m->int_or("rot_dim", 0);
      h.dim = dim + h.rot_part;
      h.vdim = (int)m->int_or("vdim", dim);
      h.kv_rank = (int)m->int_or("kv_rank", 0);
      h.q_rank = (int)m->int_or("q_rank", 0);
      h.scale = (float)m->num_or("scale", 1.0);
      h.rot_dims = h.rot_part;
      if (const Json* r = m->get("rot")) if (r->is_obj()) { h.rot_dims = (int)r->int_or("dims", h.rot_part); h.rot_base = r->num_or("base", 10000.0); }
      if (h.heads <= 0 || dim < 0 || h.dim <= 0 || h.vdim <= 0 || h.kv_rank <= 0 || h.q_rank < 0 || h.rot_part < 0 || h.rot_dims < 0 || h.rot_dims > h.rot_part ||
          h.rot_dims % 2 || h.rot_base <= 0.0) { *err = "config.json: bad latent-attention sizes"; return false; }
      if (h.out_gate && h.q_rank > 0) { *err = "config.json: 'latent_attention_2' has no query latent"; return false; }
      if (!h.out_gate && h.q_rank <= 0) { *err = "config.json: 'latent_attention' needs 'q_rank'"; return false; }
    } else { *err = "config.json: unknown layer type '" + type + "' (wkv, latent_attention, latent_attention_2)"; return false; }
    if (!parse_hybrid_mlp(l, &h, err)) return false;
    if (h.mlp == HybridLayerSpec::DENSE && h.ff_limit <= 0.f) { *err = "config.json: a dense mlp needs a positive 'limit'"; return false; }
    if (h.mlp == HybridLayerSpec::MOE) {
      if (h.shared_ff > 0) { *err = "config.json: this architecture has no shared expert"; return false; }
      h.route = HybridLayerSpec::ROUTE_SOFTMAX_ALL; h.glu = HybridLayerSpec::GLU_NONE_RELU2;
    }
    own.push_back(h);
  }
  // run order: layers before the loop, the looped run `times` times, the rest
  const int n = (int)own.size();
  int start = 0, stop = 0, times = 1;
  if (const Json* lp = j.get("loop")) {
    if (lp->is_obj()) {
      start = (int)lp->int_or("start", 0); stop = (int)lp->int_or("stop", start); times = (int)lp->int_or("times", 1);
      if (start < 0 || stop < start || stop > n || times < 1) { *err = "config.json: bad 'loop'"; return false; }
    }
  }
  std::vector<int> first_run((size_t)n, -1);
  auto push = [&](int i) {
    HybridLayerSpec h = own[(size_t)i];
    h.tensor_index = i;
    if (first_run[(size_t)i] >= 0) h.weights_of = first_run[(size_t)i];
    else first_run[(size_t)i] = (int)s->hybrid.size();
    s->hybrid.push_back(h);
  };
  for (int i = 0; i < start; ++i) push(i);
  for (int t = 0; t < times; ++t) for (int i = start; i < stop; ++i) push(i);
  for (int i = stop; i < n; ++i) push(i);
  s->L = (int)s->hybrid.size();
  if (s->vocab <= 0 || s->d <= 0) { *err = "config.json misses a required size"; return false; }
  return true;
}

// Balenex: a layer list of 'parallel' mixers (windowed attention with kept first tokens, short convolutions, per-head
// q / k norm, rotary positions in halves and rotated values, beside gated linear attention) and 'attention' mixers
// (windowed attention that also sees one pooled key / value per block of older positions), gated silu feed-forwards with
// biases, and grouped RMS norms before and after every sublayer.
static bool parse_attention_sizes(const Json& m, HybridLayerSpec* h) {
  h->heads = (int)m.int_or("heads", 0); h->kv_heads = (int)m.int_or("kv_heads", h->heads);
  h->dim = (int)m.int_or("dim", 0); h->vdim = (int)m.int_or("vdim", h->dim);
  h->scale = (float)m.num_or("scale", 1.0);
  if (const Json* mk = m.get("mask")) if (mk->is_obj()) {
    h->window = (int)mk->int_or("size", 0); h->keep_first = (int)mk->int_or("keep_first", 0); h->pool = (int)mk->int_or("pool", 0);
  }
  return h->heads > 0 && h->kv_heads > 0 && h->heads % h->kv_heads == 0 && h->dim > 0 && h->vdim > 0 && h->window > 0 && h->keep_first >= 0 && h->pool >= 0;
}

static bool parse_balenex(const Json& j, ModelSpec* s, std::string* err) {
  s->model_type = "balenex";
  s->vocab = (int)j.int_or("vocab", 0);
  s->d = (int)j.int_or("width", 0);
  if (const Json* n = j.get("norm")) { s->eps = (float)n->num_or("eps", 1e-5); s->norm_groups = (int)n->int_or("groups", 1); }
  s->hyb_prenorm_pair = s->hyb_postnorm = true;
  s->max_pos = 1 << 20;                 // rotary angles are computed from the position: no table bounds them
  s->torch_dtype = "bfloat16";
  s->bos = (int)j.int_or("bos_token_id", -1);
  s->eos = (int)j.int_or("eos_token_id", -1);
  if (s->vocab <= 0 || s->d <= 0) { *err = "config.json misses a required size"; return false; }
  if (s->norm_groups < 1 || s->d % s->norm_groups) { *err = "config.json: 'norm.groups' must divide the width"; return false; }
  const Json* ls = j.get("layers");
  if (!ls || !ls->is_arr() || ls->arr.empty()) { *err = "config.json: 'layers' must be a non-empty array"; return false; }
  for (const Json& l : ls->arr) {
    HybridLayerSpec h;
    const std::string type = l.str_or("type", "");
    const Json* m = l.get("mixer");
    if (!m || !m->is_obj()) { *err = "config.json: a layer has no 'mixer'"; return false; }
    if (type == "parallel") {
      h.mixer = HybridLayerSpec::WINDOW_GLA;
      const Json *a = m->get("left"), *r = m->get("right");
      if (!a || !a->is_obj() || !r || !r->is_obj()) { *err = "config.json: a parallel mixer needs 'left' and 'right'"; return false; }
      if (!parse_attention_sizes(*a, &h) || h.pool != 0) { *err = "config.json: bad sizes of the attention side"; return false; }
      h.conv = (int)a->int_or("conv", 1);
      h.head_norm = h.rot_halves = h.v_rot = true;
      if (const Json* ro = a->get("rot")) if (ro->is_obj()) { h.rot_dims = (int)ro->int_or("dims", 0); h.rot_base = ro->num_or("base", 10000.0); }
      if (h.conv < 1 || h.conv > 16 || h.rot_dims < 0 || h.rot_dims > h.dim || h.rot_dims % 2 || h.vdim % 2 || h.rot_base <= 0.0) {
        *err = "config.json: bad conv / rotary sizes of the attention side (vdim and rot.dims are even, 1 <= conv <= 16)"; return false;
      }
      h.m_heads = (int)r->int_or("heads", 0); h.m_dim = (int)r->int_or("dim", 0); h.m_vdim = (int)r->int_or("vdim", h.m_dim);
      h.tau = (float)r->num_or("tau", 1.0);
      h.decay_rank = (int)r->int_or("decay_rank", 0);
      if (h.m_heads <= 0 || h.m_dim <= 0 || h.m_vdim <= 0 || !(h.tau > 0.f)) { *err = "config.json: bad sizes of the linear-attention side"; return false; }
    } else if (type == "attention") {
      h.mixer = HybridLayerSpec::POOLED;
      if (!parse_attention_sizes(*m, &h) || h.pool < 1 || h.keep_first != 0) { *err = "config.json: bad attention sizes (mask.size and mask.pool are positive)"; return false; }
      h.head_norm = true;
    } else { *err = "config.json: unknown layer type '" + type + "' (parallel, attention)"; return false; }
    if (!parse_hybrid_mlp(l, &h, err)) return false;
    if (h.mlp == HybridLayerSpec::MOE) { *err = "config.json: this architecture has no mixture of experts"; return false; }
    if (h.mlp == HybridLayerSpec::DENSE) h.ff_silu_bias = true;
    s->hybrid.push_back(h);
  }
  s->L = (int)s->hybrid.size();
  return true;
}

static bool parse_config(const Json& j, ModelSpec* s, std::string* err) {
  if (j.str_or("architecture", "") == "Safupel") return parse_hybrid(j, s, err);
  if (j.str_or("architecture", "") == "Balenex") return parse_balenex(j, s, err);
  if (j.str_or("architecture", "") == "Girolorn") return parse_girolorn(j, s, err);
  if (j.str_or("architecture", "") == "Zezilix") return parse_zezilix(j, s, err);
  s->model_type = j.str_or("model_type", "");
  s->vocab = (int)j.int_or("vocab_size", 0);
  s->d = (int)j.int_or("hidden_size", 0);
  s->L = (int)j.int_or("num_hidden_layers", 0);
  s->H = (int)j.int_or("num_attention_heads", 0);
  s->max_pos = (int)j.int_or("max_position_embeddings", 2048);
  s->bos = (int)j.int_or("bos_token_id", -1);
  s->torch_dtype = j.str_or("torch_dtype", j.str_or("dtype", ""));
  if (const Json* e = j.get("eos_token_id")) {
    if (e->is_num()) s->eos = (int)e->num;
    else if (e->is_arr() && !e->arr.empty() && e->arr[0].is_num()) s->eos = (int)e->arr[0].num;
  }
  if (s->model_type == "opt") {
    s->KV = s->H;
    s->ffn = (int)j.int_or("ffn_dim", 0);
    s->tied = true;
    s->eps = 1e-5f;
    if (!j.bool_or("do_layer_norm_before", true)) { *err = "OPT with do_layer_norm_before=false (opt-350m) is not supported"; return false; }
    if (j.int_or("word_embed_proj_dim", s->d) != s->d) { *err = "OPT with word_embed_proj_dim != hidden_size is not supported"; return false; }
    if (j.str_or("activation_function", "relu") != "relu") { *err = "OPT activation_function must be relu"; return false; }
  } else if (s->model_type == "llama" || s->model_type == "qwen2" || s->model_type == "qwen3") {
    // Qwen2.5 / Qwen3 (the models the reference's values files deploy, ref:values-01-minimal-example2.yaml:8,
    // ...example8.yaml:8) share Llama's graph: vllm:model_executor/models/qwen2.py:160-175, qwen3.py:142-160
    const bool qwen = s->model_type != "llama";
    s->qkv_bias = s->model_type == "qwen2";
    s->qk_norm = s->model_type == "qwen3";
    s->KV = (int)j.int_or("num_key_value_heads", s->H);
    s->ffn = (int)j.int_or("intermediate_size", 0);
    s->tied = j.bool_or("tie_word_embeddings", false);
    s->eps = (float)j.num_or("rms_norm_eps", qwen ? 1e-6 : 1e-5);
    s->rope_theta = j.num_or("rope_theta", qwen ? 1000000.0 : 10000.0);
    if (const Json* rp = j.get("rope_parameters"))
      if (rp->is_obj()) s->rope_theta = rp->num_or("rope_theta", s->rope_theta);
    if (const Json* rs = j.get("rope_scaling")) {
      if (rs->is_obj()) {
        std::string t = rs->str_or("rope_type", rs->str_or("type", ""));
        if (t == "llama3") {
          s->rope_factor = rs->num_or("factor", 8.0);
          s->rope_low = rs->num_or("low_freq_factor", 1.0);
          s->rope_high = rs->num_or("high_freq_factor", 4.0);
          s->rope_orig_max = (int)rs->int_or("original_max_position_embeddings", 8192);
        } else if (!t.empty() && t != "default") {
          *err = "rope_scaling type '" + t + "' is not supported (llama3 only)";
          return false;
        }
      }
    }
    if (!qwen && (j.bool_or("attention_bias", false) || j.bool_or("mlp_bias", false))) { *err = "llama with attention_bias/mlp_bias is not supported"; return false; }
    if (s->model_type == "qwen3" && j.bool_or("attention_bias", false)) { *err = "qwen3 with attention_bias is not supported"; return false; }
    if (j.bool_or("use_sliding_window", false)) { *err = "sliding-window attention is not supported"; return false; }
  } else {
    *err = "unsupported model_type '" + s->model_type + "' (opt, llama, qwen2, qwen3)";
    return false;
  }
  if (s->H <= 0 || s->d <= 0 || s->L <= 0 || s->vocab <= 0 || s->ffn <= 0) { *err = "config.json misses a required size"; return false; }
  s->hd = (int)j.int_or("head_dim", s->d / s->H);
  if (s->hd != 64 && s->hd != 128) { *err = "head_dim must be 64 or 128"; return false; }
  if (s->H % s->KV != 0) { *err = "num_attention_heads must be a multiple of num_key_value_heads"; return false; }
  return true;
}

bool ModelDir::open(const std::string& dir, std::string* err) {
  std::string txt;
  if (!read_file(dir + "/config.json", &txt)) { *err = "cannot read " + dir + "/config.json"; return false; }
  Json cfg;
  std::string perr;
  if (!json_parse(txt, &cfg, &perr)) { *err = "config.json: " + perr; return false; }
  if (!parse_config(cfg, &spec_, err)) return false;

  std::vector<std::string> files;
  if (DIR* d = opendir(dir.c_str())) {
    while (dirent* e = readdir(d)) {
      std::string n = e->d_name;
      if (n.size() > 12 && n.substr(n.size() - 12) == ".safetensors") files.push_back(dir + "/" + n);
    }
    closedir(d);
  }
  std::sort(files.begin(), files.end());
  for (auto& path : files) {
    int fd = ::open(path.c_str(), O_RDONLY);
    if (fd < 0) { *err = "cannot open " + path; return false; }
    struct stat st;
    fstat(fd, &st);
    if (st.st_size < 8) { close(fd); *err = path + ": too small"; return false; }
    void* base = mmap(nullptr, st.st_size, PROT_READ, MAP_PRIVATE, fd, 0);
    close(fd);
    if (base == MAP_FAILED) { *err = "mmap failed for " + path; return false; }
    maps_.push_back({base, (size_t)st.st_size});
    const uint8_t* p = (const uint8_t*)base;
    uint64_t hlen;
    memcpy(&hlen, p, 8);
    if (hlen > (uint64_t)st.st_size - 8) { /* compared this way round: 8 + hlen could wrap */ *err = path + ": bad header length"; return false; }
    Json hdr;
    JsonParser jp((const char*)p + 8, hlen);
    if (!jp.parse(&hdr, &perr) || !hdr.is_obj()) { *err = path + ": header " + perr; return false; }
    const uint8_t* data0 = p + 8 + hlen;
    const uint64_t data_len = st.st_size - 8 - hlen;
    for (auto& kv : hdr.obj) {
      if (kv.first == "__metadata__") continue;
      const Json& t = kv.second;
      const Json* off = t.get("data_offsets");
      const Json* shp = t.get("shape");
      if (!off || !shp || off->arr.size() != 2) { *err = path + ": bad entry " + kv.first; return false; }
      HostTensor ht;
      ht.dtype = t.str_or("dtype", "");
      for (auto& s : shp->arr) ht.shape.push_back((int64_t)s.num);
      const uint64_t b = (uint64_t)off->arr[0].num, e = (uint64_t)off->arr[1].num;
      const int esz = (ht.dtype == "F32" || ht.dtype == "I32") ? 4 : 2;
      if (e > data_len || b > e || (e - b) != (uint64_t)ht.numel() * esz) { *err = path + ": bad offsets for " + kv.first; return false; }
      if (ht.dtype != "BF16" && ht.dtype != "F16" && ht.dtype != "F32" && ht.dtype != "I32") { *err = kv.first + ": dtype " + ht.dtype + " unsupported"; return false; }
      ht.data = data0 + b;
      tensors_[kv.first] = ht;
    }
  }
  return true;
}

const HostTensor* ModelDir::find(const std::string& name) const {
  auto it = tensors_.find(name);
  return it == tensors_.end() ? nullptr : &it->second;
}

static inline uint16_t f32_bf16(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x40);
  u += 0x7fffu + ((u >> 16) & 1u);
  return (uint16_t)(u >> 16);
}
static inline float f16_f32(uint16_t h) {
  const uint32_t sign = (uint32_t)(h & 0x8000) << 16;
  uint32_t exp = (h >> 10) & 0x1f, man = h & 0x3ff, u;
  if (exp == 0) {
    if (man == 0) u = sign;
    else {
      exp = 127 - 15 + 1;
      while (!(man & 0x400)) { man <<= 1; --exp; }
      u = sign | (exp << 23) | ((man & 0x3ff) << 13);
    }
  } else if (exp == 31) u = sign | 0x7f800000u | (man << 13);
  else u = sign | ((exp + 127 - 15) << 23) | (man << 13);
  float f;
  memcpy(&f, &u, 4);
  return f;
}

static inline float bf16_f32(uint16_t b) {
  const uint32_t u = (uint32_t)b << 16;
  float f;
  memcpy(&f, &u, 4);
  return f;
}

bool ModelDir::read_16(const std::string& name, int64_t r0, int64_t r1, int64_t c0, int64_t c1, bool f16,
                       std::vector<uint16_t>* out, std::string* err) const {
  const HostTensor* t = find(name);
  if (!t) { *err = "missing tensor " + name; return false; }
  if (t->dtype == "I32") { *err = name + ": an integer table cannot be read as a 16-bit float tensor"; return false; }
  int64_t rows, cols;
  if (t->shape.size() == 1) { rows = t->shape[0]; cols = 1; c0 = 0; c1 = 1; }
  else if (t->shape.size() == 2) { rows = t->shape[0]; cols = t->shape[1]; }
  else { *err = name + ": rank must be 1 or 2"; return false; }
  if (r1 < 0) r1 = rows;
  if (c1 < 0) c1 = cols;
  if (r0 < 0 || r1 > rows || c0 < 0 || c1 > cols || r0 > r1 || c0 > c1) {
    *err = name + ": slice out of range (shape " + std::to_string(rows) + "x" + std::to_string(cols) + ")";
    return false;
  }
  const int64_t nr = r1 - r0, nc = c1 - c0;
  out->resize((size_t)(nr * nc));
  for (int64_t r = 0; r < nr; ++r) {
    const int64_t src = (r0 + r) * cols + c0;
    uint16_t* dst = out->data() + r * nc;
    if (t->dtype == (f16 ? "F16" : "BF16")) {
      memcpy(dst, t->data + src * 2, (size_t)nc * 2);
    } else if (t->dtype == "F16") {
      const uint16_t* s = (const uint16_t*)t->data + src;
      for (int64_t c = 0; c < nc; ++c) dst[c] = f32_bf16(f16_f32(s[c]));
    } else if (t->dtype == "BF16") {
      const uint16_t* s = (const uint16_t*)t->data + src;
      for (int64_t c = 0; c < nc; ++c) dst[c] = f32_to_f16_bits(bf16_f32(s[c]));
    } else {
      const float* s = (const float*)t->data + src;
      for (int64_t c = 0; c < nc; ++c) dst[c] = f16 ? f32_to_f16_bits(s[c]) : f32_bf16(s[c]);
    }
  }
  return true;
}

bool ModelDir::read_f32(const std::string& name, std::vector<float>* out, std::string* err) const {
  const HostTensor* t = find(name);
  if (!t) { *err = "missing tensor " + name; return false; }
  const int64_t n = t->numel();
  out->resize((size_t)n);
  if (t->dtype == "F32") memcpy(out->data(), t->data, (size_t)n * 4);
  else if (t->dtype == "I32") { const int32_t* s = (const int32_t*)t->data; for (int64_t i = 0; i < n; ++i) (*out)[i] = (float)s[i]; }
  else {
    const uint16_t* s = (const uint16_t*)t->data;
    for (int64_t i = 0; i < n; ++i) (*out)[i] = t->dtype == "BF16" ? bf16_f32(s[i]) : f16_f32(s[i]);
  }
  return true;
}

}  // namespace kge

// ---------------------------------------------------------------- host-only C view (tests, tooling)
#include "common.cuh"
#include "kge.h"

struct kge_model_dir { kge::ModelDir md; };

extern "C" kge_model_dir* kge_model_open(const char* dir) {
  if (!dir) { kge::set_error("kge_model_open: null directory"); return nullptr; }
  auto* m = new kge_model_dir();
  std::string err;
  if (!m->md.open(dir, &err)) { kge::set_error("kge_model_open: %s", err.c_str()); delete m; return nullptr; }
  return m;
}
extern "C" void kge_model_close(kge_model_dir* m) { delete m; }

extern "C" int kge_model_spec_json(const kge_model_dir* m, char* out, int cap) {
  KGE_REQUIRE(m && out && cap > 0, "kge_model_spec_json: bad arguments");
  const kge::ModelSpec& s = m->md.spec();
  if (s.is_hybrid()) {
    std::string j = "{\"model_type\":\"" + s.model_type + "\",\"vocab\":" + std::to_string(s.vocab) + ",\"d\":" + std::to_string(s.d) +
                    ",\"L\":" + std::to_string(s.L) + ",\"has_weights\":" + (m->md.has_weights() ? "true" : "false") + ",\"layers\":[";
    char buf[2048];
    for (size_t i = 0; i < s.hybrid.size(); ++i) {
      const kge::HybridLayerSpec& h = s.hybrid[i];
      snprintf(buf, sizeof buf,
               "%s{\"mixer\":%d,\"width\":%d,\"blocks\":%d,\"conv\":%d,\"heads\":%d,\"kv_heads\":%d,\"dim\":%d,\"vdim\":%d,\"chunk\":%d,"
               "\"scale\":%.9g,\"left_scale\":%.9g,\"right_scale\":%.9g,\"m_heads\":%d,\"m_dim\":%d,\"m_vdim\":%d,\"gate_cap\":%.9g,"
               "\"mlp\":%d,\"ff\":%d,\"experts\":%d,\"top\":%d,\"expert_ff\":%d,\"shared_ff\":%d,\"softcap\":%.9g,\"rot_dims\":%d,\"rot_base\":%.17g,"
               "\"yarn_factor\":%.17g,\"yarn_original\":%.17g,\"yarn_fast\":%.17g,\"yarn_slow\":%.17g,\"route\":%d,\"glu\":%d,\"expert_limit\":%.9g,"
               "\"shared_limit\":%.9g,\"weights_of\":%d,\"tensor_index\":%d,\"q_rank\":%d,\"kv_rank\":%d,\"rot_part\":%d,\"out_gate\":%d,"
               "\"decay_rank\":%d,\"ff_limit\":%.9g,\"router_scale\":%.9g,\"window\":%d,\"keep_first\":%d,\"pool\":%d,\"tau\":%.9g,"
               "\"head_norm\":%d,\"rot_halves\":%d,\"v_rot\":%d,\"ff_silu_bias\":%d}",
               i ? "," : "", h.mixer, h.width, h.blocks, h.conv, h.heads, h.kv_heads, h.dim, h.vdim, h.chunk, (double)h.scale, (double)h.left_scale,
               (double)h.right_scale, h.m_heads, h.m_dim, h.m_vdim, (double)h.gate_cap, h.mlp, h.ff, h.experts, h.top, h.expert_ff, h.shared_ff,
               (double)h.softcap, h.rot_dims, h.rot_base, h.yarn_factor, h.yarn_original, h.yarn_fast, h.yarn_slow, h.route, h.glu, (double)h.expert_limit,
               (double)h.shared_limit, h.weights_of, h.tensor_index < 0 ? (int)i : h.tensor_index, h.q_rank, h.kv_rank, h.rot_part, h.out_gate ? 1 : 0,
               h.decay_rank, (double)h.ff_limit, (double)h.router_scale, h.window, h.keep_first, h.pool, (double)h.tau, h.head_norm ? 1 : 0,
               h.rot_halves ? 1 : 0, h.v_rot ? 1 : 0, h.ff_silu_bias ? 1 : 0);
      j += buf;
    }
    snprintf(buf, sizeof buf, "],\"eps\":%.9g,\"logit_scale\":%.9g,\"logit_softcap\":%.9g,\"streams\":%d,\"residual_mult\":%.9g,\"embed_norm\":%s,"
             "\"norm_groups\":%d,\"postnorm\":%s}", (double)s.eps,
             (double)s.logit_scale, (double)s.logit_softcap, s.streams, (double)s.residual_mult, s.embed_norm ? "true" : "false", s.norm_groups,
             s.hyb_postnorm ? "true" : "false");
    j += buf;
    KGE_REQUIRE((int)j.size() < cap, "kge_model_spec_json: buffer of %d bytes too small", cap);
    memcpy(out, j.c_str(), j.size() + 1);
    return (int)j.size();
  }
  const int n = snprintf(out, (size_t)cap,
                         "{\"model_type\":\"%s\",\"qkv_bias\":%s,\"qk_norm\":%s,\"vocab\":%d,\"d\":%d,\"L\":%d,\"H\":%d,\"KV\":%d,\"hd\":%d,"
                         "\"ffn\":%d,\"max_pos\":%d,\"eps\":%.9g,\"tied\":%s,\"rope_theta\":%.17g,\"rope_factor\":%.17g,\"rope_low\":%.17g,"
                         "\"rope_high\":%.17g,\"rope_orig_max\":%d,\"bos\":%d,\"eos\":%d,\"has_weights\":%s}",
                         s.model_type.c_str(), s.qkv_bias ? "true" : "false", s.qk_norm ? "true" : "false", s.vocab, s.d, s.L, s.H, s.KV,
                         s.hd, s.ffn, s.max_pos, (double)s.eps, s.tied ? "true" : "false", s.rope_theta, s.rope_factor, s.rope_low,
                         s.rope_high, s.rope_orig_max, s.bos, s.eos, m->md.has_weights() ? "true" : "false");
  KGE_REQUIRE(n > 0 && n < cap, "kge_model_spec_json: buffer of %d bytes too small", cap);
  return n;
}

static int64_t model_read_16(const kge_model_dir* m, const char* name, int64_t r0, int64_t r1, int64_t c0, int64_t c1, bool f16,
                             uint16_t* out, int64_t cap);
extern "C" int64_t kge_model_read_bf16(const kge_model_dir* m, const char* name, int64_t r0, int64_t r1, int64_t c0, int64_t c1,
                                       uint16_t* out, int64_t cap) {
  return model_read_16(m, name, r0, r1, c0, c1, false, out, cap);
}
extern "C" int64_t kge_model_read_f16(const kge_model_dir* m, const char* name, int64_t r0, int64_t r1, int64_t c0, int64_t c1,
                                      uint16_t* out, int64_t cap) {
  return model_read_16(m, name, r0, r1, c0, c1, true, out, cap);
}
static int64_t model_read_16(const kge_model_dir* m, const char* name, int64_t r0, int64_t r1, int64_t c0, int64_t c1, bool f16,
                             uint16_t* out, int64_t cap) {
  if (!m || !name || !out) { kge::set_error("kge_model_read_bf16: null argument"); return -1; }
  std::vector<uint16_t> v;
  std::string err;
  if (!m->md.read_16(name, r0, r1, c0, c1, f16, &v, &err)) { kge::set_error("kge_model_read_bf16: %s", err.c_str()); return -1; }
  if ((int64_t)v.size() > cap) { kge::set_error("kge_model_read_bf16: %lld elements > capacity %lld", (long long)v.size(), (long long)cap); return -1; }
  memcpy(out, v.data(), v.size() * 2);
  return (int64_t)v.size();
}
