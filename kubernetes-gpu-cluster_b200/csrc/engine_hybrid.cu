// Layer-list ("hybrid") models in the engine: a config.json that lists its layers, each with a token mixer (gated
// linear recurrence, attention and a matrix memory side by side, attention alone with rotary positions, a soft cap
// and sink logits, a WKV recurrence, attention through latents, windowed attention with kept first tokens beside gated
// linear attention, or windowed attention over pooled blocks) and a feed-forward (dense or mixture of experts),
// reading ONE norm of an fp32 residual stream, a norm each in sequence (optionally with a norm of each result as
// well), or a norm each of a hyper-connected residual (several copies of the stream).  This file loads such a model (weights in the engine's storage
// type, fused where one activation feeds several projections), sizes its arena, paged caches and recurrent-state pool,
// and runs its step: the same flattened batch, block tables and slot mapping as every other model, plus a state slot
// per request.  Nothing here depends on how a prompt was cut into steps: recurrences continue from the slot, attention
// reads the paged cache, and every other operation is per row.
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <algorithm>

#include "engine.h"
#include "hybrid_ops.h"

using namespace kge;

namespace kge {
inline namespace b16 {
// attn.cu: the paged attention of the Llama family (tcgen05 kernel for steps with query chunks, TMA-staged split-KV
// kernels for decode steps; 64- and 128-wide heads, bfloat16) with an optional soft cap and sink logits
int paged_attn_extras(void* out, const void* q, int q_stride, const void* k_cache, const void* v_cache, const int32_t* block_table,
                      int max_blocks_per_seq, const int32_t* seq_lens, const int32_t* query_start_loc, int B, int T, int max_q_len,
                      int max_seq_len, int H, int KV, int hd, int block_size, float scale, float softcap, const float* sinks, void* workspace,
                      int64_t workspace_bytes, void* stream);
bool paged_attn_extras_decode_ok(int B, int H, int KV, int hd, int block_size);
// attn_tc.cu: the tcgen05 prompt kernel with a sliding window and kept first tokens or pooled blocks (64- / 128-wide heads)
bool paged_attn_window_tc_ok(int H, int KV, int hd, int vd, int bs, int pool, int pool_slots);
int paged_attn_window_tc(void* out, const void* q, int q_stride, const void* kc, const void* vc, const void* pkc, const void* pvc, const int32_t* bt,
                         int max_blocks, const int32_t* sl, const int32_t* qsl, int B, int max_q_len, int H, int KV, int hd, int bs, float scale,
                         int window, int keep_first, int pool, int pool_slots, cudaStream_t st);
// gemm_tc.cu: one tcgen05 launch over row groups padded to 256 (the experts of a prompt step)
int gemm_grouped(void* y, const void* x, const void* w, int T, int N, int K, int groups, const int32_t* tile_group, int glu, float glu_alpha,
                 float glu_limit, cudaStream_t st);
// gemm_tc.cu: silu(x w[:f]^T + b[:f]) * (x w[f:]^T + b[f:]) with the pair formed in the epilogue; f a multiple of 64, K of 8
int gemm_silu_gate_bias(void* y, const void* x, const void* w_gate_up, const void* bias_gate_up, int T, int f, int K, cudaStream_t st);
}

namespace {

struct HB {
  kge_engine* e;
  const ModelDir* md;
  int64_t dummy_seed;
  uint64_t counter = 1;
  std::string err;
  bool dummy() const { return !md->has_weights(); }
  int esz() const { return e->f32 ? 4 : 2; }

  void* dalloc(int64_t elems, int bytes_per) {
    void* p = nullptr;
    if (cudaMalloc(&p, (size_t)std::max<int64_t>(elems, 8) * bytes_per) != cudaSuccess) {
      err = std::string("cudaMalloc failed: ") + cudaGetErrorString(cudaGetLastError());
      return nullptr;
    }
    e->allocs.push_back(p);
    return p;
  }
  void* upload(const std::vector<float>& v) {
    void* p = dalloc((int64_t)v.size(), esz());
    if (!p) return nullptr;
    e->weight_bytes += (int64_t)v.size() * esz();
    cudaError_t ce;
    if (e->f32) ce = cudaMemcpy(p, v.data(), v.size() * 4, cudaMemcpyHostToDevice);
    else {
      std::vector<uint16_t> h(v.size());
      for (size_t i = 0; i < v.size(); ++i) {            // round to nearest even (exact for bfloat16 checkpoints)
        uint32_t u; memcpy(&u, &v[i], 4);
        if ((u & 0x7fffffffu) > 0x7f800000u) h[i] = (uint16_t)((u >> 16) | 0x40);
        else { u += 0x7fffu + ((u >> 16) & 1u); h[i] = (uint16_t)(u >> 16); }
      }
      ce = cudaMemcpy(p, h.data(), h.size() * 2, cudaMemcpyHostToDevice);
    }
    if (ce != cudaSuccess) { err = "cudaMemcpy of weights failed"; return nullptr; }
    return p;
  }
  // arrays kept in one type whatever the engine's storage type (sink logits, rotary frequencies)
  template <typename T>
  T* upload_raw(const std::vector<T>& v) {
    T* p = (T*)dalloc((int64_t)v.size(), sizeof(T));
    if (!p) return nullptr;
    e->weight_bytes += (int64_t)v.size() * sizeof(T);
    if (cudaMemcpy(p, v.data(), v.size() * sizeof(T), cudaMemcpyHostToDevice) != cudaSuccess) { err = "cudaMemcpy of weights failed"; return nullptr; }
    return p;
  }
  float* vec_f32(const std::string& name, int64_t n, float dummy_const) {
    std::vector<float> v((size_t)n, dummy_const);
    if (!dummy() && !stack({name}, {n}, 1, &v)) return nullptr;
    return upload_raw(v);
  }
  // a vector that a checkpoint may leave out (null then: the caller's default); without a checkpoint the given values
  float* opt_f32(const std::string& name, int64_t n, const std::vector<float>& dummy_v, bool* failed) {
    if (dummy()) return dummy_v.empty() ? nullptr : upload_raw(dummy_v);
    if (!md->find(name)) return nullptr;
    std::vector<float> v;
    if (!stack({name}, {n}, 1, &v)) { *failed = true; return nullptr; }
    return upload_raw(v);
  }
  // tensors stacked along their first dimension; every one must have `inner` elements per leading index
  bool stack(const std::vector<std::string>& names, const std::vector<int64_t>& lead, int64_t inner, std::vector<float>* out) {
    out->clear();
    for (size_t i = 0; i < names.size(); ++i) {
      const HostTensor* t = md->find(names[i]);
      if (!t) { err = "missing tensor " + names[i]; return false; }
      if (t->numel() != lead[i] * inner || (inner > 1 && t->shape.size() >= 2 && t->shape.back() != inner && t->shape.size() == 2)) {
        err = names[i] + ": checkpoint shape does not match config.json (expected " + std::to_string(lead[i]) + " x " + std::to_string(inner) + ")";
        return false;
      }
      std::vector<float> v;
      if (!md->read_f32(names[i], &v, &err)) return false;
      out->insert(out->end(), v.begin(), v.end());
    }
    return true;
  }
  // a matrix [sum(lead), K] (rows stacked), or random / constant values for a model without a checkpoint
  void* mat(const std::vector<std::string>& names, const std::vector<int64_t>& lead, int64_t inner, float dummy_scale, float dummy_const = 0.f) {
    int64_t rows = 0;
    for (auto l : lead) rows += l;
    if (dummy()) {
      if (e->f32) { err = "random weights are made in bfloat16 only"; return nullptr; }
      void* p = dalloc(rows * inner, 2);
      if (!p) return nullptr;
      e->weight_bytes += rows * inner * 2;
      if (dummy_scale > 0.f) fill_uniform(p, rows * inner, (uint64_t)dummy_seed * 0x100000001B3ull + (counter++) * 0x9E3779B9ull, dummy_scale, false, e->stream);
      else fill_const(p, rows * inner, dummy_const, false, e->stream);
      return p;
    }
    std::vector<float> v;
    if (!stack(names, lead, inner, &v)) return nullptr;
    return upload(v);
  }
};

int64_t align_up64(int64_t v, int64_t a) { return (v + a - 1) / a * a; }

}  // namespace

int hybrid_engine_build(kge_engine* e, const ModelDir& md, int64_t dummy_seed, std::string* err) {
  const ModelSpec& s = e->spec;
  HB b{e, &md, dummy_seed};
  const int d = s.d;
  auto fail = [&](const std::string& m) { *err = m; return -1; };
  const float ws = 0.02f * 1.7320508f;
#define HB_OK(p) do { if (!(p)) return fail(b.err); } while (0)
  HB_OK(e->embed = (bf16*)b.mat({"embed"}, {s.vocab}, d, ws));
  HB_OK(e->lm_head = (bf16*)b.mat({"head"}, {s.vocab}, d, ws));
  const bool plain_norm_w = s.hyb_layernorm || s.streams > 0 || s.hyb_postnorm;      // the norm weight multiplies as it is (else it is applied as 1 + w)
  HB_OK(e->final_w = (bf16*)b.mat({"final.norm"}, {d}, 1, 0.f, plain_norm_w ? 1.f : 0.f));
  if (s.embed_norm) HB_OK(e->embed_norm_w = b.mat({"embed.norm"}, {d}, 1, 0.f, 1.f));
  e->hyb.resize(s.L);
  int64_t state_floats = 0;
  int max_mo = 1;
  int max_proj = 1, max_mix = 1, max_ff = 1, max_gate = 1, max_u = 1, max_top = 0, max_eff = 1, max_E = 1;
  int max_hd = 0, max_qr = 0, max_kvr = 0, max_lkv = 0, max_lq = 0;      // WKV heads * dim; latent ranks, [k | v] and query widths
  int max_mix2 = 0;
  for (int i = 0; i < s.L; ++i) {
    const HybridLayerSpec& h = s.hybrid[i];
    HybridLayerW& L = e->hyb[i];
    const std::string p = "l" + std::to_string(h.tensor_index >= 0 ? h.tensor_index : i) + ".", mx = p + "mix.", fp = p + "mlp.";
    if (h.weights_of >= 0) {                   // another layer's tensors; the paged caches below and the state stay this layer's own
      L = e->hyb[h.weights_of];
      L.kc = L.vc = L.pkc = L.pvc = nullptr;
      L.state_off = state_floats;
      if (h.mixer == HybridLayerSpec::RGLRU) state_floats += rglru_state_floats(h.width, h.conv);
      else if (h.mixer == HybridLayerSpec::PARALLEL) state_floats += mlstm_state_floats(h.m_heads, h.m_dim, h.m_vdim);
      else if (h.mixer == HybridLayerSpec::WKV) state_floats += wkv_state_floats(d, h.heads, h.dim);
      else if (h.mixer == HybridLayerSpec::WINDOW_GLA)
        state_floats += short_conv_state_floats((h.heads + h.kv_heads) * h.dim + h.kv_heads * h.vdim, h.conv) + gla_state_floats(h.m_heads, h.m_dim, h.m_vdim);
      continue;
    }
    const float norm_one = plain_norm_w ? 1.f : 0.f;      // the weight that leaves the normed row as it is
    HB_OK(L.norm1 = b.mat({p + "norm1"}, {d}, 1, 0.f, norm_one));
    if (s.hyb_prenorm_pair && h.mlp != HybridLayerSpec::NONE) HB_OK(L.norm2 = b.mat({p + "norm2"}, {d}, 1, 0.f, norm_one));
    if (s.hyb_postnorm) {
      HB_OK(L.norm1b = b.mat({p + "norm1b"}, {d}, 1, 0.f, 1.f));
      if (h.mlp != HybridLayerSpec::NONE) HB_OK(L.norm2b = b.mat({p + "norm2b"}, {d}, 1, 0.f, 1.f));
    }
    L.state_off = state_floats;
    if (h.mixer == HybridLayerSpec::RGLRU) {
      const int w = h.width, bw = w / h.blocks;
      L.yx.N = 2 * w; L.yx.K = d;
      HB_OK(L.yx.w = b.mat({mx + "y", mx + "x"}, {w, w}, d, ws));
      HB_OK(L.yx.b = b.mat({mx + "y.b", mx + "x.b"}, {w, w}, 1, 0.f, 0.f));
      HB_OK(L.conv_w = b.mat({mx + "conv"}, {w}, h.conv, 0.3f));
      HB_OK(L.conv_b = b.mat({mx + "conv.b"}, {w}, 1, 0.f, 0.f));
      L.ra.N = bw; L.ra.K = bw; L.ri.N = bw; L.ri.K = bw;
      HB_OK(L.ra.w = b.mat({mx + "ra"}, {(int64_t)h.blocks * bw}, bw, 0.1f));
      HB_OK(L.ra.b = b.mat({mx + "ra.b"}, {w}, 1, 0.f, 0.f));
      HB_OK(L.ri.w = b.mat({mx + "ri"}, {(int64_t)h.blocks * bw}, bw, 0.1f));
      HB_OK(L.ri.b = b.mat({mx + "ri.b"}, {w}, 1, 0.f, 0.f));
      HB_OK(L.lam = b.mat({mx + "lam"}, {w}, 1, 0.f, -1.0f));
      L.o.N = d; L.o.K = w;
      HB_OK(L.o.w = b.mat({mx + "o"}, {d}, w, ws));
      state_floats += rglru_state_floats(w, h.conv);
      max_proj = std::max(max_proj, 2 * w); max_mix = std::max(max_mix, w); max_gate = std::max(max_gate, 2 * w); max_u = std::max(max_u, w);
    } else if (h.mixer == HybridLayerSpec::ATTENTION) {
      const int nq = h.heads * h.dim, nk = h.kv_heads * h.dim;
      if (!h.v_from_k) return fail("an attention mixer with a value projection of its own is not built");
      L.qk.N = nq + nk; L.qk.K = d;
      HB_OK(L.qk.w = b.mat({mx + "q", mx + "k"}, {nq, nk}, d, ws));
      if (h.qk_norm) {
        HB_OK(L.q_norm = b.mat({mx + "q.norm"}, {nq}, 1, 0.f, 1.f));
        HB_OK(L.k_norm = b.mat({mx + "k.norm"}, {nk}, 1, 0.f, 1.f));
      }
      if (h.sink) HB_OK(L.sinks = b.vec_f32(mx + "sink", h.heads, 0.f));
      if (h.rot_dims > 0) {
        std::vector<double> fr((size_t)h.rot_dims / 2);
        rotary_frequencies(h.rot_dims, h.rot_base, h.yarn_factor, h.yarn_original, h.yarn_fast, h.yarn_slow, fr.data(), &L.rot_mult);
        HB_OK(L.rot_freq = b.upload_raw(fr));
      }
      L.o.N = d; L.o.K = h.heads * h.vdim;
      HB_OK(L.o.w = b.mat({mx + "o"}, {d}, h.heads * h.vdim, ws));
      max_proj = std::max(max_proj, L.qk.N); max_mix = std::max(max_mix, L.o.K);
    } else if (h.mixer == HybridLayerSpec::WINDOW_GLA) {
      const int nq = h.heads * h.dim, nk = h.kv_heads * h.dim, nv = h.kv_heads * h.vdim, mk = h.m_heads * h.m_dim, mv = h.m_heads * h.m_vdim;
      const std::string a = mx + "left.", r = mx + "right.";
      int lr = h.decay_rank;
      if (!b.dummy()) {
        const HostTensor* t1 = md.find(r + "a1");
        if (!t1 || t1->shape.size() != 2) return fail("missing tensor " + r + "a1");
        lr = (int)t1->shape[0];
      } else if (lr <= 0) lr = 16;
      L.off_k = nq; L.off_v = nq + nk; L.off_mq = L.off_v + nv; L.off_mk = L.off_mq + mk; L.off_mv = L.off_mk + mk; L.off_mg = L.off_mv + mv; L.off_a1 = L.off_mg + mv;
      L.proj.N = L.off_a1 + lr; L.proj.K = d;
      HB_OK(L.proj.w = b.mat({a + "q", a + "k", a + "v", r + "q", r + "k", r + "v", r + "g", r + "a1"}, {nq, nk, nv, mk, mk, mv, mv, lr}, d, ws));
      if (b.dummy()) HB_OK(L.proj.b = b.mat({}, {L.proj.N}, 1, 0.f, 0.f));
      else {
        std::vector<float> bias;      // the attention side's projections carry biases, the other side's do not
        if (!b.stack({a + "q.b", a + "k.b", a + "v.b"}, {nq, nk, nv}, 1, &bias)) return fail(b.err);
        bias.resize((size_t)L.proj.N, 0.f);
        HB_OK(L.proj.b = b.upload(bias));
      }
      HB_OK(L.conv_w = b.mat({a + "q.conv", a + "k.conv", a + "v.conv"}, {nq, nk, nv}, h.conv, 0.5f));
      HB_OK(L.q_norm = b.mat({a + "q.norm"}, {h.dim}, 1, 0.f, 1.f));
      HB_OK(L.k_norm = b.mat({a + "k.norm"}, {h.dim}, 1, 0.f, 1.f));
      if (h.rot_dims > 0) {
        std::vector<double> fr((size_t)h.rot_dims / 2);
        rotary_frequencies(h.rot_dims, h.rot_base, 0.0, 0.0, 32.0, 1.0, fr.data(), &L.rot_mult);
        HB_OK(L.rot_freq = b.upload_raw(fr));
      }
      if (h.v_rot) {
        std::vector<double> fr((size_t)h.vdim / 2);
        float one;
        rotary_frequencies(h.vdim, h.rot_base, 0.0, 0.0, 32.0, 1.0, fr.data(), &one);
        HB_OK(L.v_freq = b.upload_raw(fr));
      }
      L.o.N = d; L.o.K = h.heads * h.vdim;
      HB_OK(L.o.w = b.mat({a + "o"}, {d}, L.o.K, ws));
      L.o2.N = d; L.o2.K = mv;
      HB_OK(L.o2.w = b.mat({r + "o"}, {d}, mv, ws));
      L.wkv_w2.N = mk; L.wkv_w2.K = lr;
      HB_OK(L.wkv_w2.w = b.mat({r + "a2"}, {mk}, lr, ws));
      HB_OK(L.wkv_w2.b = b.mat({r + "a2.b"}, {mk}, 1, 0.f, 2.f));
      {
        // the per-head norm of the read-out: one weight of m_vdim numbers, laid out once per head
        std::vector<std::string> rep((size_t)h.m_heads, r + "norm");
        std::vector<int64_t> lead((size_t)h.m_heads, h.m_vdim);
        HB_OK(L.wkv_norm = b.mat(rep, lead, 1, 0.f, 1.f));
      }
      HB_OK(L.side_norm[0] = b.mat({a + "out"}, {d}, 1, 0.f, 1.f));
      HB_OK(L.side_norm[1] = b.mat({r + "out"}, {d}, 1, 0.f, 1.f));
      state_floats += short_conv_state_floats(nq + nk + nv, h.conv) + gla_state_floats(h.m_heads, h.m_dim, h.m_vdim);
      max_proj = std::max(max_proj, L.proj.N); max_u = std::max(max_u, nq + nk + nv); max_mix = std::max(max_mix, L.o.K); max_mix2 = std::max(max_mix2, mv);
      max_gate = std::max(max_gate, mk); max_mo = std::max(max_mo, mv);
    } else if (h.mixer == HybridLayerSpec::POOLED) {
      const int nq = h.heads * h.dim, nk = h.kv_heads * h.dim, nv = h.kv_heads * h.vdim;
      L.off_k = nq; L.off_v = nq + nk;
      L.proj.N = nq + nk + nv; L.proj.K = d;
      HB_OK(L.proj.w = b.mat({mx + "q", mx + "k", mx + "v"}, {nq, nk, nv}, d, ws));
      HB_OK(L.proj.b = b.mat({mx + "q.b", mx + "k.b", mx + "v.b"}, {nq, nk, nv}, 1, 0.f, 0.f));
      L.o.N = d; L.o.K = h.heads * h.vdim;
      HB_OK(L.o.w = b.mat({mx + "o"}, {d}, L.o.K, ws));
      HB_OK(L.o.b = b.mat({mx + "o.b"}, {d}, 1, 0.f, 0.f));
      max_proj = std::max(max_proj, L.proj.N); max_mix = std::max(max_mix, L.o.K);
    } else if (h.mixer == HybridLayerSpec::WKV) {
      const int hd = h.heads * h.dim;
      int lr = h.decay_rank;
      if (!b.dummy()) {
        const HostTensor* t1 = md.find(mx + "w1");
        if (!t1 || t1->shape.size() != 2) return fail("missing tensor " + mx + "w1");
        lr = (int)t1->shape[0];
      } else if (lr <= 0) lr = 64;
      HB_OK(L.wkv_mu = b.mat({mx + "mu.r", mx + "mu.k", mx + "mu.v", mx + "mu.g", mx + "mu.w"}, {d, d, d, d, d}, 1, 0.f, 0.5f));
      L.wkv_rkvg.N = hd; L.wkv_rkvg.K = d;
      HB_OK(L.wkv_rkvg.w = b.mat({mx + "r", mx + "k", mx + "v", mx + "g"}, {hd, hd, hd, hd}, d, ws));
      L.wkv_w1.N = lr; L.wkv_w1.K = d; L.wkv_w2.N = hd; L.wkv_w2.K = lr;
      HB_OK(L.wkv_w1.w = b.mat({mx + "w1"}, {lr}, d, ws));
      HB_OK(L.wkv_w2.w = b.mat({mx + "w2"}, {hd}, lr, ws));
      HB_OK(L.wkv_w2.b = b.mat({mx + "w0"}, {hd}, 1, 0.f, -1.f));
      HB_OK(L.wkv_u = b.vec_f32(mx + "u", hd, 0.5f));
      HB_OK(L.wkv_norm = b.mat({mx + "norm"}, {hd}, 1, 0.f, 1.f));
      L.o.N = d; L.o.K = hd;
      HB_OK(L.o.w = b.mat({mx + "o"}, {d}, hd, ws));
      state_floats += wkv_state_floats(d, h.heads, h.dim);
      max_hd = std::max(max_hd, hd); max_mix = std::max(max_mix, hd); max_gate = std::max(max_gate, hd); max_mo = std::max(max_mo, hd); max_u = std::max(max_u, lr);
    } else if (h.mixer == HybridLayerSpec::LATENT) {
      const int nope = h.dim - h.rot_part, nq = h.heads * h.dim, nkv = h.kv_rank + h.rot_part, nv = h.heads * h.vdim;
      if (h.q_rank > 0) {
        L.lat_dkv = h.q_rank; L.proj.N = h.q_rank + nkv; L.proj.K = d;
        HB_OK(L.proj.w = b.mat({mx + "dq", mx + "dkv"}, {h.q_rank, nkv}, d, ws));
        HB_OK(L.lat_qnorm = b.mat({mx + "dq.norm"}, {h.q_rank}, 1, 0.f, 1.f));
        L.lat_uq.N = nq; L.lat_uq.K = h.q_rank;
        HB_OK(L.lat_uq.w = b.mat({mx + "uq"}, {nq}, h.q_rank, ws * 4));
      } else {
        L.lat_dkv = nq; L.lat_g = nq + nkv; L.proj.N = nq + nkv + (h.out_gate ? nv : 0); L.proj.K = d;
        if (h.out_gate) HB_OK(L.proj.w = b.mat({mx + "q", mx + "dkv", mx + "g"}, {nq, nkv, nv}, d, ws));
        else HB_OK(L.proj.w = b.mat({mx + "q", mx + "dkv"}, {nq, nkv}, d, ws));
      }
      HB_OK(L.lat_kvnorm = b.mat({mx + "dkv.norm"}, {h.kv_rank}, 1, 0.f, 1.f));
      L.lat_ukv.N = h.heads * nope + nv; L.lat_ukv.K = h.kv_rank;
      HB_OK(L.lat_ukv.w = b.mat({mx + "uk", mx + "uv"}, {h.heads * nope, nv}, h.kv_rank, ws * 4));
      if (h.rot_dims > 0) {
        std::vector<double> fr((size_t)h.rot_dims / 2);
        rotary_frequencies(h.rot_dims, h.rot_base, 0.0, 0.0, 32.0, 1.0, fr.data(), &L.rot_mult);
        HB_OK(L.rot_freq = b.upload_raw(fr));
      }
      L.o.N = d; L.o.K = nv;
      HB_OK(L.o.w = b.mat({mx + "o"}, {d}, nv, ws));
      max_proj = std::max(max_proj, L.proj.N); max_mix = std::max(max_mix, nv);
      max_qr = std::max(max_qr, h.q_rank); max_kvr = std::max(max_kvr, h.kv_rank); max_lkv = std::max(max_lkv, L.lat_ukv.N); max_lq = std::max(max_lq, nq);
    } else {
      const int nq = h.heads * h.dim, nk = h.kv_heads * h.dim, nv = h.kv_heads * h.vdim, mq = h.m_heads * h.m_dim, mv = h.m_heads * h.m_vdim;
      L.off_k = nq; L.off_v = nq + nk; L.off_mq = L.off_v + nv; L.off_mk = L.off_mq + mq; L.off_mv = L.off_mk + mq; L.off_mg = L.off_mv + mv;
      L.proj.N = L.off_mg + mv; L.proj.K = d;
      const std::string a = mx + "left.", r = mx + "right.";
      HB_OK(L.proj.w = b.mat({a + "q", a + "k", a + "v", r + "q", r + "k", r + "v", r + "g"}, {nq, nk, nv, mq, mq, mv, mv}, d, ws));
      L.gates.N = 2 * h.m_heads; L.gates.K = d;
      HB_OK(L.gates.w = b.mat({r + "i", r + "f"}, {h.m_heads, h.m_heads}, d, ws));
      HB_OK(L.gates.b = b.mat({r + "i.b", r + "f.b"}, {h.m_heads, h.m_heads}, 1, 0.f, 1.f));
      HB_OK(L.m_norm = b.mat({r + "norm"}, {mv}, 1, 0.f, 1.f));
      // one output projection over [attention | matrix memory]: rows of the two matrices side by side
      const int ka = h.heads * h.vdim, ko = ka + mv;
      L.o2.N = d; L.o2.K = ko;
      if (b.dummy()) HB_OK(L.o2.w = b.mat({}, {d}, ko, ws));
      else {
        std::vector<float> lo, ro, cat((size_t)d * ko);
        if (!b.stack({a + "o"}, {d}, ka, &lo) || !b.stack({r + "o"}, {d}, mv, &ro)) return fail(b.err);
        for (int n = 0; n < d; ++n) {
          memcpy(&cat[(size_t)n * ko], &lo[(size_t)n * ka], (size_t)ka * 4);
          memcpy(&cat[(size_t)n * ko + ka], &ro[(size_t)n * mv], (size_t)mv * 4);
        }
        HB_OK(L.o2.w = b.upload(cat));
      }
      state_floats += mlstm_state_floats(h.m_heads, h.m_dim, h.m_vdim);
      max_mo = std::max(max_mo, mv);
      max_proj = std::max(max_proj, L.proj.N); max_mix = std::max(max_mix, ko); max_gate = std::max(max_gate, 2 * h.m_heads);
    }
    if (s.streams > 0) {
      // the hyper-connection tensors and the per-column scales of both sublayers (a checkpoint without them: plain sums)
      const int S = s.streams;
      bool bad = false;
      for (int q = 0; q < (h.mlp == HybridLayerSpec::NONE ? 1 : 2); ++q) {
        const std::string hc = p + "hc" + std::to_string(q + 1) + ".";
        std::vector<float> din((size_t)S, 1.f / S), dout((size_t)S, 1.f), dmix((size_t)S * S, 0.f), dls((size_t)d, 1.f);
        for (int a1 = 0; a1 < S; ++a1) for (int a2 = 0; a2 < S; ++a2) dmix[(size_t)a1 * S + a2] = a1 == a2 ? 0.75f : 0.25f / std::max(S - 1, 1);
        L.hc_in[q] = b.opt_f32(hc + "in", S, din, &bad);
        L.hc_out[q] = b.opt_f32(hc + "out", S, dout, &bad);
        L.hc_mix[q] = b.opt_f32(hc + "mix", (int64_t)S * S, dmix, &bad);
        L.col_scale[q] = b.opt_f32(p + "ls" + std::to_string(q + 1), d, dls, &bad);
        if (bad || !b.err.empty()) return fail(b.err);
      }
    }
    if (h.mlp == HybridLayerSpec::DENSE && h.ff_silu_bias) {
      // silu(gate h + b) * (up h + b), then down with its bias: [gate | up] rows and biases in one block
      L.up.N = 2 * h.ff; L.up.K = d; L.down.N = d; L.down.K = h.ff;
      HB_OK(L.ff_gate = b.mat({fp + "gate", fp + "up"}, {h.ff, h.ff}, d, ws));
      HB_OK(L.ff_gate_b = b.mat({fp + "gate.b", fp + "up.b"}, {h.ff, h.ff}, 1, 0.f, 0.f));
      L.up.w = L.ff_gate; L.up.b = L.ff_gate_b;
      HB_OK(L.down.w = b.mat({fp + "down"}, {d}, h.ff, ws));
      HB_OK(L.down.b = b.mat({fp + "down.b"}, {d}, 1, 0.f, 0.f));
      max_ff = std::max(max_ff, 3 * h.ff);
    } else if (h.mlp == HybridLayerSpec::DENSE && h.ff_limit > 0.f) {
      L.up.N = h.ff; L.up.K = d; L.down.N = d; L.down.K = h.ff;
      HB_OK(L.ff_gate = b.mat({fp + "gate", fp + "up"}, {h.ff, h.ff}, d, ws));
      L.up.w = (uint8_t*)L.ff_gate + (int64_t)h.ff * d * b.esz();
      HB_OK(L.down.w = b.mat({fp + "down"}, {d}, h.ff, ws));
      max_ff = std::max(max_ff, h.ff);
    } else if (h.mlp == HybridLayerSpec::DENSE) {
      L.up.N = h.ff; L.up.K = d; L.down.N = d; L.down.K = h.ff;
      HB_OK(L.up.w = b.mat({fp + "up"}, {h.ff}, d, ws));
      HB_OK(L.down.w = b.mat({fp + "down"}, {d}, h.ff, ws));
      max_ff = std::max(max_ff, h.ff);
    } else if (h.mlp == HybridLayerSpec::MOE) {
      L.router.N = h.experts; L.router.K = d;
      HB_OK(L.router.w = b.mat({fp + "router"}, {h.experts}, d, ws * 4));
      if (h.router_bias) HB_OK(L.router_b = b.mat({fp + "router.b"}, {h.experts}, 1, 0.f, 0.f));
      // per expert [gate | up] rows in one block (what the fused gated GEMM reads), then all experts' down matrices
      std::vector<std::string> gu, dn;
      const bool gated = h.glu != HybridLayerSpec::GLU_NONE_RELU2;      // an ungated expert has one front matrix: [E, ff, d]
      std::vector<int64_t> lf((size_t)(gated ? 2 : 1) * h.experts, h.expert_ff), ld((size_t)h.experts, d);
      for (int x = 0; x < h.experts; ++x) {
        const std::string ep = fp + "e" + std::to_string(x) + ".";
        if (gated) gu.push_back(ep + "gate");
        gu.push_back(ep + "up"); dn.push_back(ep + "down");
      }
      HB_OK(L.e_gate = b.mat(gu, lf, d, ws));
      L.e_up = gated ? (uint8_t*)L.e_gate + (int64_t)h.expert_ff * d * b.esz() : nullptr;
      HB_OK(L.e_down = b.mat(dn, ld, h.expert_ff, ws));
      if (h.shared_ff > 0) {
        L.s_gate.N = L.s_up.N = h.shared_ff; L.s_gate.K = L.s_up.K = d; L.s_down.N = d; L.s_down.K = h.shared_ff;
        // [gate | up] in one matrix: what the fused gated GEMM reads; the generic kernel takes the two halves
        HB_OK(L.s_gate.w = b.mat({fp + "shared.gate", fp + "shared.up"}, {h.shared_ff, h.shared_ff}, d, ws));
        L.s_up.w = (uint8_t*)L.s_gate.w + (int64_t)h.shared_ff * d * b.esz();
        HB_OK(L.s_down.w = b.mat({fp + "shared.down"}, {d}, h.shared_ff, ws));
        if (h.shared_gate) HB_OK(L.s_sg = b.mat({fp + "shared.sg"}, {1}, d, ws));
        max_ff = std::max(max_ff, h.shared_ff);
      }
      max_top = std::max(max_top, h.top); max_eff = std::max(max_eff, h.expert_ff); max_E = std::max(max_E, h.experts);
    }
  }
#undef HB_OK
  e->slot_stride = std::max<int64_t>(state_floats, 1);

  const int Tm = e->cfg.max_num_batched_tokens, Rm = e->cfg.max_num_seqs, es = b.esz();
  // 16-bit logits rows: straight out of the tensor-core GEMM when its shapes allow (then the row stride is the
  // vocabulary), else converted from fp32 into rows padded to the samplers' 16-byte alignment
  e->hyb_head_tc = !e->f32 && s.vocab % 8 == 0 && d % 8 == 0;
  e->ld_logits = e->hyb_head_tc ? s.vocab : (int)align_up64(s.vocab, 64);
  e->vocab_shard = e->vocab_loc = s.vocab; e->vocab_col0 = 0;
  auto aalloc = [&](int64_t elems, int esz) -> void* { return b.dalloc(elems, esz); };
  e->res32 = (float*)aalloc((int64_t)Tm * d * std::max(s.streams, 1), 4);
  if (s.streams > 0) { e->y32 = (float*)aalloc((int64_t)Tm * d, 4); if (!e->y32) return fail(b.err); }
  if (max_hd > 0) {
    e->mixes = aalloc((int64_t)5 * Tm * d, es); e->rkvg = aalloc((int64_t)4 * Tm * max_hd, es);
    if (!e->mixes || !e->rkvg) return fail(b.err);
  }
  if (max_lkv > 0) {
    e->latq = aalloc((int64_t)Tm * std::max(max_qr, 1), es); e->latc = aalloc((int64_t)Tm * max_kvr, es);
    e->latkv = aalloc((int64_t)Tm * max_lkv, es); e->qbuf = aalloc((int64_t)Tm * max_lq, es);
    if (!e->latq || !e->latc || !e->latkv || !e->qbuf) return fail(b.err);
  }
  e->hx = aalloc((int64_t)Tm * d, es);
  e->pbuf = aalloc((int64_t)Tm * max_proj, es);
  e->ubuf = aalloc((int64_t)Tm * max_u, es);
  e->mixbuf = aalloc((int64_t)Tm * max_mix, es);
  if (max_mix2 > 0) { e->mixbuf2 = aalloc((int64_t)Tm * max_mix2, es); if (!e->mixbuf2) return fail(b.err); }
  e->obuf1 = aalloc((int64_t)Tm * d, es);
  e->obuf2 = aalloc((int64_t)Tm * d, es);
  e->ffbuf = aalloc((int64_t)Tm * max_ff, es);
  e->gates32 = (float*)aalloc((int64_t)Tm * max_gate, 4);
  e->mo32 = (float*)aalloc((int64_t)Tm * max_mo, 4);
  e->hsel = aalloc((int64_t)std::max(Rm, Tm) * d, es);
  // logits rows: the sampled rows of a step, or every row a trace asks for
  e->logits32 = (float*)aalloc((int64_t)std::max(Rm, Tm) * s.vocab, 4);
  e->logits = (bf16*)aalloc((int64_t)std::max(Rm, Tm) * e->ld_logits, 2);
  e->state = (float*)aalloc((int64_t)Rm * e->slot_stride, 4);
  if (max_top > 0) {
    const int64_t np0 = (int64_t)Tm * max_top;
    const int64_t np = e->f32 ? np0 : (np0 / 256 + max_E + 1) * 256;      // bfloat16: room for groups padded to 256 rows
    e->moe_rows_padded = np;
    e->moe_tile_group = (int32_t*)aalloc(np / 256 + 1, 4);
    if (!e->moe_tile_group) return fail(b.err);
    e->moe_hidden = aalloc(np * max_eff, es);
    e->moe_out = aalloc(np * d, es);
    if (!e->f32) {
      e->moe_xperm = aalloc(np * d, 2); e->moe_operm = aalloc(np * d, 2);
      if (!e->moe_xperm || !e->moe_operm || cudaMallocHost((void**)&e->moe_goff_host, (size_t)(max_E + 1) * 4) != cudaSuccess) return fail("expert staging allocation failed: " + b.err);
    }
    e->moe_goff = (int32_t*)aalloc(max_E + 1, 4);
    e->moe_ptok = (int32_t*)aalloc(np, 4); e->moe_pdest = (int32_t*)aalloc(np, 4); e->moe_cexp = (int32_t*)aalloc(np, 4);
    e->moe_pw = (float*)aalloc(np, 4); e->moe_cw = (float*)aalloc(np, 4);
    if (!e->moe_hidden || !e->moe_out || !e->moe_goff || !e->moe_ptok || !e->moe_pdest || !e->moe_cexp || !e->moe_pw || !e->moe_cw) return fail(b.err);
  }
  {
    // split-KV scratch of the TMA-staged decode attention, for attention mixers whose heads it takes
    int64_t need = 0;
    for (auto& h : s.hybrid)
      if ((h.mixer == HybridLayerSpec::ATTENTION || h.mixer == HybridLayerSpec::LATENT) && !e->f32 && (h.dim == 64 || h.dim == 128) && h.vdim == h.dim)
        need = std::max<int64_t>(need, kge_attn_workspace_bytes(Rm, h.heads, h.dim, e->cfg.max_model_len));
    if (need > 0) {
      e->ws_attn_bytes = need;
      e->ws_attn = aalloc(need, 1);
      if (!e->ws_attn) return fail("attention workspace allocation failed: " + b.err);
    }
  }
  e->d_out = (int32_t*)aalloc(Rm, 4);
  e->lp_vals = (float*)aalloc((int64_t)Rm * 21, 4);
  e->lp_ids = (int32_t*)aalloc((int64_t)Rm * 21, 4);
  e->lp_rank = (int32_t*)aalloc(Rm, 4);
  e->mask_pairs = (int32_t*)aalloc(2 * kge_engine::kMaxMaskPairs, 4);
  e->max_blocks_per_seq = (e->cfg.max_model_len + e->cfg.block_size - 1) / e->cfg.block_size;
  carve_meta(nullptr, Tm, Rm, std::max(Rm, Tm), e->max_blocks_per_seq, &e->meta_bytes);
  e->meta_dev = (uint8_t*)aalloc(e->meta_bytes, 1);
  if (!e->res32 || !e->hx || !e->pbuf || !e->ubuf || !e->mixbuf || !e->obuf1 || !e->obuf2 || !e->ffbuf || !e->gates32 || !e->mo32 || !e->hsel ||
      !e->logits32 || !e->logits || !e->state || !e->d_out || !e->lp_vals || !e->lp_ids || !e->lp_rank || !e->mask_pairs || !e->meta_dev)
    return fail("activation arena allocation failed: " + b.err);
  if (cudaMallocHost((void**)&e->meta_host, e->meta_bytes) != cudaSuccess ||
      cudaMallocHost((void**)&e->out_host, (size_t)Rm * 4) != cudaSuccess ||
      cudaMallocHost((void**)&e->lp_vals_host, (size_t)Rm * 21 * 4) != cudaSuccess ||
      cudaMallocHost((void**)&e->lp_ids_host, (size_t)Rm * 21 * 4) != cudaSuccess ||
      cudaMallocHost((void**)&e->lp_rank_host, (size_t)Rm * 4) != cudaSuccess ||
      cudaMallocHost((void**)&e->mask_pairs_host, (size_t)2 * kge_engine::kMaxMaskPairs * 4) != cudaSuccess)
    return fail("pinned staging allocation failed");
  cudaMemsetAsync(e->state, 0, (size_t)Rm * e->slot_stride * 4, e->stream);

  // paged caches of the attention sides: K [blocks, G, block_size, dim], V [blocks, G, block_size, vdim] per layer
  int64_t blk_bytes = 0;
  for (auto& h : s.hybrid)
    if (h.has_cache()) blk_bytes += (int64_t)h.kv_heads * (e->cfg.block_size + (h.pool > 0 ? pool_slots_per_block(e->cfg.block_size, h.pool) : 0)) * (h.dim + h.vdim) * es;
  int nb = e->cfg.num_blocks;
  if (nb <= 0) {
    const int64_t cap = (int64_t)e->cfg.max_num_seqs * e->max_blocks_per_seq + 1;
    if (blk_bytes == 0) nb = (int)cap;
    else {
      size_t free_b = 0, total_b = 0;
      cudaMemGetInfo(&free_b, &total_b);
      const int64_t budget = (int64_t)((double)total_b * e->cfg.gpu_memory_utilization) - (int64_t)(total_b - free_b);
      nb = (int)std::min<int64_t>(std::max<int64_t>(0, budget / blk_bytes), cap);
    }
  }
  if (nb < 2) return fail("no memory left for the KV cache");
  // a request holds at most max_model_len - 1 computed tokens (the last sampled token is never fed back)
  if ((int64_t)(nb - 1) * e->cfg.block_size < e->cfg.max_model_len - 1)
    return fail("the model's max seq len (" + std::to_string(e->cfg.max_model_len) + ") is larger than the number of tokens the KV cache can hold (" +
                std::to_string((int64_t)(nb - 1) * e->cfg.block_size) + "); raise num_blocks / gpu_memory_utilization or lower max_model_len");
  e->num_blocks = nb;
  e->kv_bytes = blk_bytes * nb;
  for (int i = 0; i < s.L; ++i) {
    const HybridLayerSpec& h = s.hybrid[i];
    if (!h.has_cache()) continue;
    const int64_t nk = (int64_t)nb * h.kv_heads * e->cfg.block_size * h.dim, nv = (int64_t)nb * h.kv_heads * e->cfg.block_size * h.vdim;
    e->hyb[i].kc = aalloc(nk, es); e->hyb[i].vc = aalloc(nv, es);
    if (!e->hyb[i].kc || !e->hyb[i].vc) return fail("KV pool allocation failed");
    cudaMemsetAsync(e->hyb[i].kc, 0, (size_t)nk * es, e->stream);
    cudaMemsetAsync(e->hyb[i].vc, 0, (size_t)nv * es, e->stream);
    if (h.pool > 0) {
      // one pooled key / value per block of `pool` positions, on the same pages: entry b of a request lives in its page b / slots
      const int ps = pool_slots_per_block(e->cfg.block_size, h.pool);
      const int64_t pk = (int64_t)nb * h.kv_heads * ps * h.dim, pv = (int64_t)nb * h.kv_heads * ps * h.vdim;
      e->hyb[i].pkc = aalloc(pk, es); e->hyb[i].pvc = aalloc(pv, es);
      if (!e->hyb[i].pkc || !e->hyb[i].pvc) return fail("pooled KV pool allocation failed");
      cudaMemsetAsync(e->hyb[i].pkc, 0, (size_t)pk * es, e->stream);
      cudaMemsetAsync(e->hyb[i].pvc, 0, (size_t)pv * es, e->stream);
    }
  }
  SchedConfig sc;
  sc.max_num_seqs = e->cfg.max_num_seqs;
  sc.max_num_batched_tokens = e->cfg.max_num_batched_tokens;
  sc.max_model_len = e->cfg.max_model_len;
  sc.block_size = e->cfg.block_size;
  sc.num_blocks = nb;
  sc.enable_chunked_prefill = e->cfg.enable_chunked_prefill != 0;
  sc.eos_token_id = s.eos;
  sc.num_state_slots = e->cfg.max_num_seqs;        // every running request owns a slot of the recurrent-state pool
  e->sched.reset(new Scheduler(sc));
  if (cudaStreamSynchronize(e->stream) != cudaSuccess) return fail(std::string("device error during initialisation: ") + cudaGetErrorString(cudaGetLastError()));
  return 0;
}

enum { C_GEMM_S = 0, C_GEMM_L = 1, C_ATT_DEC = 2, C_ATT_GEN = 3, C_NORM = 4, C_KVW = 5, C_ACT = 6, C_EMBED = 7, C_SAMPLE = 8, C_RGLRU = 10, C_MLSTM = 11, C_MOE = 12 };

// KGE_TRACE_LAUNCHES=1 (diagnostics): synchronise after every launch of a step and name it on stderr
static const bool g_trace_launches = getenv("KGE_TRACE_LAUNCHES") != nullptr;
#define HFWD(cat, bytes, flops, call)      \
  do {                                     \
    timer_begin(e, cat, bytes, flops);     \
    int _rc = (call);                      \
    if (_rc) return _rc;                   \
    timer_end(e);                          \
    ++e->launches;                         \
    if (g_trace_launches) {                \
      fprintf(stderr, "[kge] %s ...", #call); fflush(stderr);                                 \
      const cudaError_t _ce = cudaStreamSynchronize(e->stream);                                \
      fprintf(stderr, " %s\n", cudaGetErrorString(_ce)); fflush(stderr);                       \
    }                                      \
  } while (0)

// y[T, N] = act(x[T, K] w^T + b) in the engine's storage type (fp32 output where asked).  bfloat16 engines send every
// shape the tensor-core GEMM takes (16-byte rows, packed operands) there; the rest, and float32 engines, run the
// shape-agnostic kernel.
static int dense(kge_engine* e, void* y, int ldy, const void* x, int ldx, const HybMat& m, int T, int act, bool out_f32 = false) {
  if (!e->f32 && !out_f32 && m.K % 8 == 0 && ldx == m.K && ldy == m.N && (act == ACT_NONE || act == ACT_GELU_ERF) &&
      ((uintptr_t)x & 15) == 0 && ((uintptr_t)m.w & 15) == 0)
    return kge_gemm_bf16(y, x, m.w, m.b, T, m.N, m.K, act == ACT_GELU_ERF ? 3 : 0, nullptr, 0, e->stream);
  LinearArgs a;
  a.x = x; a.ldx = ldx; a.w = m.w; a.bias = m.b; a.y = y; a.ldy = ldy; a.T = T; a.N = m.N; a.K = m.K; a.act = act;
  a.elt = e->f32 ? KGE_ELT_F32 : KGE_ELT_BF16; a.out_f32 = out_f32 || e->f32;
  return linear_any(a, e->stream);
}
#define DENSE(y, ldy, x, ldx, m, T, act)                                                                    \
  HFWD((T) <= 256 ? C_GEMM_S : C_GEMM_L, es * ((double)(m).N * (m).K + (double)(T) * ((m).K + (m).N)), \
       2.0 * (T) * (double)(m).N * (m).K, dense(e, y, ldy, x, ldx, m, T, act))

int hybrid_forward(kge_engine* e, int T, int B, int R, int max_blocks, const StepMeta& m, bool any_random) {
  const ModelSpec& s = e->spec;
  const int d = s.d, elt = e->f32 ? KGE_ELT_F32 : KGE_ELT_BF16, bs = e->cfg.block_size;
  const double es = e->f32 ? 4 : 2;
  cudaStream_t st = e->stream;
  auto at = [&](void* base, int64_t elems) -> void* { return (uint8_t*)base + elems * (int64_t)es; };
  const double Td = (double)T * d;
  // keys a query sees, summed over the step's rows, for the attention roofline: host-side copy of the step's layout
  const uint8_t* hostm = e->meta_host;
  const StepMeta hm = carve_meta(const_cast<uint8_t*>(hostm), T, B, R, max_blocks, nullptr);
  bool decode_only = true;
  for (int i = 0; i < B; ++i) decode_only &= hm.qsl[i + 1] - hm.qsl[i] == 1;
  // Steps that carry prompt pieces run their kernels in plain stream order: they are tens of milliseconds long, early
  // launch buys nothing there, and hundreds of long-running CTAs of one kernel waiting on the previous one would only
  // hold shared memory.  Decode steps keep programmatic dependent launch (and run as CUDA graphs).
  struct PdlOff { bool on; explicit PdlOff(bool o) : on(o) { if (on) pdl_suspend(true); } ~PdlOff() { if (on) pdl_suspend(false); } } pdl_off(!decode_only);
  // the model's norm of residual rows: RMS with the weight applied as 1 + w, or the weight-only layer norm
  auto layer_norm = [&](void* y, const int32_t* rows, const void* w, int R, float out_scale) -> int {
    if (s.hyb_postnorm) return group_rmsnorm_f32in(y, e->res32, rows, w, R, d, s.norm_groups, s.eps, out_scale, elt, st);
    return s.hyb_layernorm ? layernorm_f32in(y, e->res32, rows, w, R, d, s.eps, out_scale, elt, st)
                           : rmsnorm_f32in(y, e->res32, rows, w, R, d, s.eps, 1.f, out_scale, elt, st);
  };
  // hyper-connected residual: S streams per token, read through a sublayer's input weights and a norm, written back
  // through its mix matrix and output weights; designs with one plain stream keep the residual sum
  const bool hyper = s.streams > 0;
  const int S = std::max(s.streams, 1);
  auto stream_read = [&](void* y, const float* in_w, const int32_t* rows, const void* w, int R, float out_scale, float* sum_out) -> int {
    StreamNormArgs sn;
    sn.y = y; sn.xs = e->res32; sn.in_w = in_w; sn.rows = rows; sn.w = w; sn.sum_out = sum_out; sn.R = R; sn.d = d; sn.S = S; sn.eps = s.eps; sn.out_scale = out_scale; sn.elt = elt;
    return stream_norm(sn, st);
  };
  if (hyper) HFWD(C_EMBED, Td * (es + 4.0 * S), 0, embed_norm_streams(e->res32, m.ids, e->embed, s.embed_norm ? e->embed_norm_w : nullptr, T, d, S, s.eps, elt, st));
  else HFWD(C_EMBED, Td * (es + 4), 0, embed_f32(e->res32, m.ids, e->embed, T, d, elt, st));
  bool hx_ready = false;      // the previous layer's last write of the streams already formed this layer's normed input
  for (int i = 0; i < s.L; ++i) {
    const HybridLayerSpec& h = s.hybrid[i];
    const HybridLayerW& L = e->hyb[i];
    if (hyper) { if (!hx_ready) HFWD(C_NORM, Td * (4.0 * S + es), 0, stream_read(e->hx, L.hc_in[0], nullptr, L.norm1, T, 1.f, nullptr)); hx_ready = false; }
    else if (!hx_ready) HFWD(C_NORM, Td * (4 + es), 0, layer_norm(e->hx, nullptr, L.norm1, T, 1.f));
    hx_ready = false;
    CombineArgs cb;
    const void* inner_w[2] = {nullptr, nullptr};      // a norm of a source's own before the sources are summed (models with normed results)
    bool y32_used = false;
    int sub = 0;                                       // the sublayer whose result is being summed (0: mixer, 1: feed-forward)
    auto add_src = [&](const void* p, int ld, float scale, const float* rscale = nullptr, int rs_stride = 0) {
      cb.src[cb.n] = p; cb.ld[cb.n] = ld; cb.scale[cb.n] = scale; cb.rscale[cb.n] = rscale; cb.rs_stride[cb.n] = rs_stride; ++cb.n;
    };
    // more sources follow: a plain stream takes them as they come; with several streams they gather in an fp32 row first
    auto flush_more = [&]() -> int {
      if (cb.n == 0) return 0;
      int rc;
      if (!hyper) rc = residual_combine(e->res32, cb, T, d, elt, st);
      else {
        if (!y32_used) { KGE_CUDA_OK(cudaMemsetAsync(e->y32, 0, (size_t)T * d * 4, st)); y32_used = true; }
        rc = residual_combine(e->y32, cb, T, d, elt, st);
      }
      cb = CombineArgs();
      return rc;
    };
    // the write of the streams also forms the next sublayer's normed input (the feed-forward's, or the next layer's mixer's)
    auto flush = [&]() -> int {
      if (s.hyb_postnorm) {
        // the sublayer's result through its own norm into the stream, and the next sublayer's normed input in the same pass
        PostNormArgs pa;
        pa.res = e->res32; pa.nsrc = cb.n; pa.src_scale = cb.scale[0]; pa.T = T; pa.d = d; pa.groups = s.norm_groups; pa.eps = s.eps; pa.elt = elt;
        for (int q = 0; q < cb.n && q < 2; ++q) { pa.src[q] = cb.src[q]; pa.ld[q] = cb.ld[q]; pa.inner_w[q] = inner_w[q]; }
        pa.post_w = sub == 0 ? L.norm1b : L.norm2b;
        if (sub == 0 && h.mlp != HybridLayerSpec::NONE) { pa.next_w = L.norm2; pa.next_y = e->hx; }
        else if (i + 1 < s.L) { pa.next_w = e->hyb[i + 1].norm1; pa.next_y = e->hx; hx_ready = true; }
        cb = CombineArgs(); inner_w[0] = inner_w[1] = nullptr;
        return postnorm_residual(pa, st);
      }
      if (!hyper) return flush_more();
      StreamCombineArgs sc;
      sc.xs = e->res32; sc.src = cb; sc.y32 = y32_used ? e->y32 : nullptr; sc.col_scale = L.col_scale[sub]; sc.mix = L.hc_mix[sub]; sc.out_w = L.hc_out[sub];
      sc.mult = s.residual_mult; sc.T = T; sc.d = d; sc.S = S; sc.elt = elt; sc.eps = s.eps;
      const bool mixer_done = sub == 0 && h.mlp != HybridLayerSpec::NONE;
      if (mixer_done) { sc.next_in = L.hc_in[1]; sc.next_w = L.norm2; sc.next_y = e->hx; }
      else if (i + 1 < s.L) { sc.next_in = e->hyb[i + 1].hc_in[0]; sc.next_w = e->hyb[i + 1].norm1; sc.next_y = e->hx; hx_ready = true; }
      cb = CombineArgs(); y32_used = false;
      return stream_combine(sc, st);
    };
    if (h.mixer == HybridLayerSpec::RGLRU) {
      const int w = h.width, bw = w / h.blocks;
      DENSE(e->pbuf, 2 * w, e->hx, d, L.yx, T, ACT_NONE);
      RglruArgs ra;
      ra.yx = e->pbuf; ra.u = e->ubuf; ra.gates = e->gates32; ra.out = e->mixbuf;
      ra.conv_w = L.conv_w; ra.conv_b = L.conv_b; ra.lam = L.lam;
      ra.state = e->state + L.state_off; ra.slot_stride = e->slot_stride;
      ra.slots = m.sslot; ra.qsl = m.qsl; ra.positions = m.pos; ra.token_req = m.treq;
      ra.B = B; ra.T = T; ra.width = w; ra.taps = h.conv; ra.decay_c = 8.f; ra.elt = elt;
      const double Tw = (double)T * w;
      HFWD(C_RGLRU, Tw * 2 * es, 0, rglru_conv(ra, st));
      for (int gsel = 0; gsel < 2; ++gsel) {           // block-diagonal gate projections of u, kept in fp32
        const HybMat& gm = gsel ? L.ri : L.ra;
        LinearArgs a;
        a.x = e->ubuf; a.ldx = w; a.w = gm.w; a.bias = gm.b; a.y = e->gates32 + (int64_t)gsel * w; a.ldy = 2 * w;
        a.T = T; a.N = bw; a.K = bw; a.nz = h.blocks; a.x_zs = bw; a.w_zs = (int64_t)bw * bw; a.b_zs = bw; a.y_zs = bw;
        a.elt = elt; a.out_f32 = true;
        HFWD(C_RGLRU, Tw * (es + 4) + (double)w * bw * es, 2.0 * Tw * bw, linear_any(a, st));
      }
      HFWD(C_RGLRU, Tw * (3 * es + 8) + 2.0 * B * rglru_state_floats(w, h.conv) * 4, 0, rglru_scan(ra, st));
      DENSE(e->obuf1, d, e->mixbuf, w, L.o, T, ACT_NONE);
      add_src(e->obuf1, d, 1.f);
    } else if (h.mixer == HybridLayerSpec::ATTENTION) {
      const int nq = h.heads * h.dim, ldp = L.qk.N, ko = L.o.K;
      DENSE(e->pbuf, ldp, e->hx, d, L.qk, T, ACT_NONE);
      RotaryArgs ro;     // norm over the whole q and k projections, rotation, K cache <- rotated keys, V cache <- the raw key projection
      ro.q = e->pbuf; ro.ldq = ldp; ro.k = at(e->pbuf, nq); ro.ldk = ldp; ro.q_norm_w = L.q_norm; ro.k_norm_w = L.k_norm; ro.eps = s.eps;
      ro.freq = L.rot_freq; ro.mult = L.rot_mult; ro.rot_dims = h.rot_dims; ro.positions = m.pos; ro.slots = m.slots;
      ro.k_cache = L.kc; ro.v_cache = L.vc; ro.T = T; ro.H = h.heads; ro.G = h.kv_heads; ro.dim = h.dim; ro.vdim = h.vdim; ro.block_size = bs; ro.elt = elt;
      HFWD(C_KVW, (double)T * (2.0 * nq + 3.0 * h.kv_heads * h.dim) * es, 0, rotary_norm_kvwrite(ro, st));
      AttnBiasArgs aa;
      aa.q = e->pbuf; aa.ldq = ldp; aa.out = e->mixbuf; aa.ldo = ko; aa.k_cache = L.kc; aa.v_cache = L.vc;
      aa.block_table = m.btab; aa.max_blocks = max_blocks; aa.seq_lens = m.seq_lens; aa.qsl = m.qsl; aa.positions = m.pos; aa.token_req = m.treq;
      aa.B = B; aa.T = T; aa.H = h.heads; aa.G = h.kv_heads; aa.dim = h.dim; aa.vdim = h.vdim; aa.block_size = bs; aa.chunk = 0;
      aa.scale = h.scale; aa.bias_span = 0.f; aa.softcap = h.softcap; aa.sinks = L.sinks; aa.elt = elt;
      for (int r = 0; r < B; ++r) aa.max_q = std::max(aa.max_q, hm.qsl[r + 1] - hm.qsl[r]);
      while (aa.num_decode < B && hm.qsl[aa.num_decode + 1] - hm.qsl[aa.num_decode] == 1) ++aa.num_decode;
      double keys = 0;                                   // visible keys over all rows
      for (int t = 0; t < T; ++t) keys += hm.pos[t] + 1;
      // steps with prompt pieces, 64- / 128-wide heads, bfloat16: the tcgen05 kernel of the Llama family (TMA-staged K/V
      // tiles, S and O in TMEM) with the cap and the sinks; everything else: the mma.sync / per-row kernels
      const bool tc = !e->f32 && (h.dim == 64 || h.dim == 128) && h.vdim == h.dim && ldp % 8 == 0 && (bs & (bs - 1)) == 0 &&
                      h.heads / h.kv_heads <= 128 && ((uintptr_t)e->pbuf & 15) == 0 &&
                      (!decode_only || (e->ws_attn && paged_attn_extras_decode_ok(B, h.heads, h.kv_heads, h.dim, bs)));
      // a decode step may be replayed as a graph while its contexts grow: sized for the longest context its block-table stride holds
      const int max_seq_bound = decode_only ? max_blocks * bs : 0;
      HFWD(decode_only ? C_ATT_DEC : C_ATT_GEN, (decode_only ? keys : (double)T) * h.kv_heads * (h.dim + h.vdim) * es + (double)T * h.heads * (h.dim + h.vdim) * es,
           2.0 * keys * h.heads * (h.dim + h.vdim),
           tc ? paged_attn_extras(e->mixbuf, e->pbuf, ldp, L.kc, L.vc, m.btab, max_blocks, m.seq_lens, m.qsl, B, T, aa.max_q, std::max(max_seq_bound, 1),
                                  h.heads, h.kv_heads, h.dim, bs, h.scale, h.softcap, L.sinks, e->ws_attn, e->ws_attn_bytes, st)
              : attn_bias_chunk(aa, st));
      DENSE(e->obuf1, d, e->mixbuf, ko, L.o, T, ACT_NONE);
      add_src(e->obuf1, d, 1.f);
    } else if (h.mixer == HybridLayerSpec::WINDOW_GLA || h.mixer == HybridLayerSpec::POOLED) {
      const bool gla = h.mixer == HybridLayerSpec::WINDOW_GLA;
      const int nq = h.heads * h.dim, nk = h.kv_heads * h.dim, nv = h.kv_heads * h.vdim, ka = h.heads * h.vdim, ldp = L.proj.N;
      DENSE(e->pbuf, ldp, e->hx, d, L.proj, T, ACT_NONE);        // every projection of the normed row in one product (biases in)
      const void* qkv = e->pbuf; int ldq = ldp;
      if (gla) {
        ShortConvArgs sc;                                        // q, k and v channels through their short convolutions
        sc.x = e->pbuf; sc.ldx = ldp; sc.y = e->ubuf; sc.ldy = nq + nk + nv; sc.w = L.conv_w; sc.C = nq + nk + nv; sc.taps = h.conv;
        sc.state = e->state + L.state_off; sc.slot_stride = e->slot_stride; sc.slots = m.sslot; sc.qsl = m.qsl; sc.positions = m.pos; sc.token_req = m.treq;
        sc.B = B; sc.T = T; sc.elt = elt;
        HFWD(C_RGLRU, (double)T * sc.C * 2 * es, 2.0 * T * sc.C * h.conv, short_conv_state(sc, st));
        ++e->launches;
        qkv = e->ubuf; ldq = sc.ldy;
      }
      HeadRotaryArgs ro;      // per-head q / k norm, rotation in halves, K cache <- keys, V cache <- values (turned by their position)
      ro.q = const_cast<void*>(qkv); ro.ldq = ldq; ro.k = at(const_cast<void*>(qkv), nq); ro.ldk = ldq; ro.v = at(const_cast<void*>(qkv), nq + nk); ro.ldv = ldq;
      ro.norm_q = ro.norm_k = h.head_norm; ro.q_norm_w = L.q_norm; ro.k_norm_w = L.k_norm; ro.eps = s.eps;
      ro.freq = L.rot_freq; ro.rot_dims = h.rot_dims; ro.v_freq = h.v_rot ? L.v_freq : nullptr; ro.positions = m.pos; ro.slots = m.slots;
      ro.k_cache = L.kc; ro.v_cache = L.vc; ro.T = T; ro.H = h.heads; ro.G = h.kv_heads; ro.dim = h.dim; ro.vdim = h.vdim; ro.block_size = bs; ro.elt = elt;
      HFWD(C_KVW, (double)T * (2.0 * nq + 2.0 * nk + 2.0 * nv) * es, 0, head_norm_rotary_kvwrite(ro, st));
      const int ps = h.pool > 0 ? pool_slots_per_block(bs, h.pool) : 0;
      if (h.pool > 0) {
        PoolKvArgs pk;       // blocks of `pool` positions that this step completes: their mean key and value
        pk.k_cache = L.kc; pk.v_cache = L.vc; pk.pk_cache = L.pkc; pk.pv_cache = L.pvc; pk.block_table = m.btab; pk.max_blocks = max_blocks;
        pk.positions = m.pos; pk.token_req = m.treq; pk.T = T; pk.G = h.kv_heads; pk.dim = h.dim; pk.vdim = h.vdim; pk.block_size = bs; pk.pool = h.pool; pk.pool_slots = ps; pk.elt = elt;
        HFWD(C_KVW, (double)T * (nk + nv) * es * (1.0 + 1.0 / h.pool), 0, pool_kv_write(pk, st));
      }
      AttnBiasArgs aa;
      aa.q = qkv; aa.ldq = ldq; aa.out = e->mixbuf; aa.ldo = ka; aa.k_cache = L.kc; aa.v_cache = L.vc;
      aa.block_table = m.btab; aa.max_blocks = max_blocks; aa.seq_lens = m.seq_lens; aa.qsl = m.qsl; aa.positions = m.pos; aa.token_req = m.treq;
      aa.B = B; aa.T = T; aa.H = h.heads; aa.G = h.kv_heads; aa.dim = h.dim; aa.vdim = h.vdim; aa.block_size = bs; aa.chunk = 0;
      aa.window = h.window; aa.keep_first = h.keep_first; aa.pool = h.pool; aa.pk_cache = L.pkc; aa.pv_cache = L.pvc; aa.pool_slots = ps;
      aa.scale = h.scale; aa.bias_span = 0.f; aa.elt = elt;
      for (int r = 0; r < B; ++r) aa.max_q = std::max(aa.max_q, hm.qsl[r + 1] - hm.qsl[r]);
      while (aa.num_decode < B && hm.qsl[aa.num_decode + 1] - hm.qsl[aa.num_decode] == 1) ++aa.num_decode;
      double keys = 0;                                   // visible keys over all rows: the window's tokens and what lies before it
      for (int t = 0; t < T; ++t) {
        const int before = std::max(hm.pos[t] - h.window + 1, 0);
        keys += std::min(hm.pos[t] + 1, h.window) + (h.pool > 0 ? before / h.pool : std::min(before, h.keep_first));
      }
      // steps with prompt pieces, 64- / 128-wide heads, bfloat16: the tcgen05 kernel (TMA-staged tiles, S and O in TMEM) with the
      // window's tile range; decode steps and everything else: the mma.sync / per-row kernels
      const bool tc = !e->f32 && !decode_only && ldq % 8 == 0 && ((uintptr_t)qkv & 15) == 0 &&
                      paged_attn_window_tc_ok(h.heads, h.kv_heads, h.dim, h.vdim, bs, h.pool, ps);
      HFWD(decode_only ? C_ATT_DEC : C_ATT_GEN, (decode_only ? keys : (double)T) * h.kv_heads * (h.dim + h.vdim) * es + (double)T * h.heads * (h.dim + h.vdim) * es,
           2.0 * keys * h.heads * (h.dim + h.vdim),
           tc ? paged_attn_window_tc(e->mixbuf, qkv, ldq, L.kc, L.vc, L.pkc, L.pvc, m.btab, max_blocks, m.seq_lens, m.qsl, B, aa.max_q, h.heads, h.kv_heads, h.dim, bs,
                                     h.scale, h.window, h.keep_first, h.pool, ps, st)
              : attn_bias_chunk(aa, st));
      if (h.v_rot) HFWD(C_ACT, (double)T * ka * 2 * es, 0, rotate_heads_halves(e->mixbuf, ka, m.pos, L.v_freq, T, h.heads, h.vdim, -1.f, elt, st));
      DENSE(e->obuf1, d, e->mixbuf, ka, L.o, T, ACT_NONE);
      if (gla) {
        const int mk = h.m_heads * h.m_dim, mv = h.m_heads * h.m_vdim, lr = L.wkv_w2.K;
        LinearArgs a2;     // the decay's logit: second half of the low-rank pair with its bias, kept in fp32
        a2.x = at(e->pbuf, L.off_a1); a2.ldx = ldp; a2.w = L.wkv_w2.w; a2.bias = L.wkv_w2.b; a2.y = e->gates32; a2.ldy = mk; a2.T = T; a2.N = mk; a2.K = lr;
        a2.elt = elt; a2.out_f32 = true;
        HFWD(C_MLSTM, es * ((double)lr * mk + (double)T * lr) + 4.0 * T * mk, 2.0 * T * (double)mk * lr, linear_any(a2, st));
        WkvArgs wa;        // gated linear attention: the state is read after the update, the decay is sigmoid(z)^(1 / tau)
        wa.d = 0; wa.r = at(e->pbuf, L.off_mq); wa.k = at(e->pbuf, L.off_mk); wa.v = at(e->pbuf, L.off_mv); wa.gate_pre = at(e->pbuf, L.off_mg); wa.ld = ldp;
        wa.decay_pre = e->gates32; wa.u = nullptr; wa.norm_w = L.wkv_norm; wa.o32 = e->mo32; wa.out = e->mixbuf2; wa.ldo = mv;
        wa.state = e->state + L.state_off + short_conv_state_floats(nq + nk + nv, h.conv); wa.slot_stride = e->slot_stride;
        wa.slots = m.sslot; wa.qsl = m.qsl; wa.positions = m.pos; wa.token_req = m.treq;
        wa.B = B; wa.T = T; wa.H = h.m_heads; wa.dim = h.m_dim; wa.vdim = h.m_vdim; wa.eps = s.eps; wa.elt = elt;
        wa.decay_mode = 1; wa.tau = h.tau; wa.read_after = true; wa.r_scale = 1.f / sqrtf((float)h.m_dim);
        for (int r = 0; r < B; ++r) wa.max_q = std::max(wa.max_q, hm.qsl[r + 1] - hm.qsl[r]);
        HFWD(C_MLSTM, 2.0 * B * gla_state_floats(h.m_heads, h.m_dim, h.m_vdim) * 4 + (double)T * ((2.0 * mk + 3.0 * mv) * es + 4.0 * mk + 8.0 * mv),
             4.0 * T * h.m_heads * (double)h.m_dim * h.m_vdim, wkv_scan(wa, st));
        ++e->launches;
        DENSE(e->obuf2, d, e->mixbuf2, mv, L.o2, T, ACT_NONE);
        // half the sum of the two sides, each RMS-normed over the width with its own weight
        add_src(e->obuf1, d, 0.5f); add_src(e->obuf2, d, 0.5f);
        inner_w[0] = L.side_norm[0]; inner_w[1] = L.side_norm[1];
      } else {
        add_src(e->obuf1, d, 1.f);
      }
    } else if (h.mixer == HybridLayerSpec::WKV) {
      const int hd = h.heads * h.dim, lr = L.wkv_w1.N;
      WkvArgs wa;
      wa.h = e->hx; wa.ldh = d; wa.mu = L.wkv_mu; wa.mixes = e->mixes; wa.nmix = 5; wa.d = d;
      wa.state = e->state + L.state_off; wa.slot_stride = e->slot_stride; wa.slots = m.sslot; wa.qsl = m.qsl; wa.positions = m.pos; wa.token_req = m.treq;
      wa.B = B; wa.T = T; wa.H = h.heads; wa.dim = h.dim; wa.eps = s.eps; wa.elt = elt;
      for (int r = 0; r < B; ++r) wa.max_q = std::max(wa.max_q, hm.qsl[r + 1] - hm.qsl[r]);
      HFWD(C_MLSTM, Td * 6 * es, 0, wkv_shift_mix(wa, st));
      ++e->launches;
      for (int z = 0; z < 4; ++z) {                      // r, k, v and the gate, each from its own blend
        HybMat mz; mz.w = at(L.wkv_rkvg.w, (int64_t)z * hd * d); mz.N = hd; mz.K = d;
        DENSE(at(e->rkvg, (int64_t)z * T * hd), hd, at(e->mixes, (int64_t)z * T * d), d, mz, T, ACT_NONE);
      }
      {
        LinearArgs a1;     // the decay's logit: a low-rank pair with a tanh between, the second half and its bias in fp32
        a1.x = at(e->mixes, (int64_t)4 * T * d); a1.ldx = d; a1.w = L.wkv_w1.w; a1.y = e->ubuf; a1.ldy = lr; a1.T = T; a1.N = lr; a1.K = d; a1.act = ACT_TANH;
        a1.elt = elt; a1.out_f32 = e->f32;
        HFWD(C_MLSTM, es * ((double)lr * d + (double)T * (d + lr)), 2.0 * Td * lr, linear_any(a1, st));
        LinearArgs a2;
        a2.x = e->ubuf; a2.ldx = lr; a2.w = L.wkv_w2.w; a2.bias = L.wkv_w2.b; a2.y = e->gates32; a2.ldy = hd; a2.T = T; a2.N = hd; a2.K = lr;
        a2.elt = elt; a2.out_f32 = true;
        HFWD(C_MLSTM, es * ((double)lr * hd + (double)T * lr) + 4.0 * T * hd, 2.0 * T * (double)hd * lr, linear_any(a2, st));
      }
      wa.r = e->rkvg; wa.k = at(e->rkvg, (int64_t)T * hd); wa.v = at(e->rkvg, (int64_t)2 * T * hd); wa.gate_pre = at(e->rkvg, (int64_t)3 * T * hd); wa.ld = hd;
      wa.decay_pre = e->gates32; wa.u = L.wkv_u; wa.norm_w = L.wkv_norm; wa.o32 = e->mo32; wa.out = e->mixbuf; wa.ldo = hd;
      HFWD(C_MLSTM, 2.0 * B * h.heads * (double)h.dim * h.dim * 4 + (double)T * hd * (5 * es + 12), 4.0 * T * h.heads * (double)h.dim * h.dim, wkv_scan(wa, st));
      ++e->launches;
      DENSE(e->obuf1, d, e->mixbuf, hd, L.o, T, ACT_NONE);
      add_src(e->obuf1, d, 1.f);
    } else if (h.mixer == HybridLayerSpec::LATENT) {
      const int H = h.heads, nope = h.dim - h.rot_part, nq = H * h.dim, nv = H * h.vdim, ldp = L.proj.N, ldkv = L.lat_ukv.N;
      DENSE(e->pbuf, ldp, e->hx, d, L.proj, T, ACT_NONE);      // [dq | dkv] or [q | dkv | g] of the normed row
      SegNormArgs sn;      // the latents' norms (fp32 statistics), written packed for the up-projections
      sn.x = e->pbuf; sn.ldx = ldp; sn.T = T; sn.eps = s.eps; sn.elt = elt; sn.nseg = 0;
      sn.col[sn.nseg] = L.lat_dkv; sn.n[sn.nseg] = h.kv_rank; sn.w[sn.nseg] = L.lat_kvnorm; sn.out[sn.nseg] = e->latc; sn.ldo[sn.nseg] = h.kv_rank; ++sn.nseg;
      if (h.q_rank > 0) { sn.col[sn.nseg] = 0; sn.n[sn.nseg] = h.q_rank; sn.w[sn.nseg] = L.lat_qnorm; sn.out[sn.nseg] = e->latq; sn.ldo[sn.nseg] = h.q_rank; ++sn.nseg; }
      HFWD(C_NORM, (double)T * (h.kv_rank + h.q_rank) * 2 * es, 0, segment_rmsnorm(sn, st));
      void* q = e->pbuf; int ldq = ldp;
      if (h.q_rank > 0) { DENSE(e->qbuf, nq, e->latq, h.q_rank, L.lat_uq, T, ACT_NONE); q = e->qbuf; ldq = nq; }
      DENSE(e->latkv, ldkv, e->latc, h.kv_rank, L.lat_ukv, T, ACT_NONE);      // every head's unrotated key part, then its value
      LatentKvArgs lk;
      lk.q = q; lk.ldq = ldq; lk.k_nope = e->latkv; lk.ldk = ldkv; lk.v = at(e->latkv, (int64_t)H * nope); lk.ldv = ldkv;
      lk.k_rot = at(e->pbuf, L.lat_dkv + h.kv_rank); lk.ldr = ldp; lk.freq = L.rot_freq; lk.rot_dims = h.rot_dims; lk.rot_part = h.rot_part;
      lk.positions = m.pos; lk.slots = m.slots; lk.k_cache = L.kc; lk.v_cache = L.vc; lk.T = T; lk.H = H; lk.dim = h.dim; lk.vdim = h.vdim; lk.block_size = bs; lk.elt = elt;
      HFWD(C_KVW, (double)T * (2.0 * H * h.rot_part + 2.0 * H * (h.dim + h.vdim)) * es, 0, latent_rotary_kvwrite(lk, st));
      AttnBiasArgs aa;
      aa.q = q; aa.ldq = ldq; aa.out = e->mixbuf; aa.ldo = nv; aa.k_cache = L.kc; aa.v_cache = L.vc;
      aa.block_table = m.btab; aa.max_blocks = max_blocks; aa.seq_lens = m.seq_lens; aa.qsl = m.qsl; aa.positions = m.pos; aa.token_req = m.treq;
      aa.B = B; aa.T = T; aa.H = H; aa.G = H; aa.dim = h.dim; aa.vdim = h.vdim; aa.block_size = bs; aa.chunk = 0;
      aa.scale = h.scale; aa.bias_span = 0.f; aa.elt = elt;
      for (int r = 0; r < B; ++r) aa.max_q = std::max(aa.max_q, hm.qsl[r + 1] - hm.qsl[r]);
      while (aa.num_decode < B && hm.qsl[aa.num_decode + 1] - hm.qsl[aa.num_decode] == 1) ++aa.num_decode;
      double keys = 0;
      for (int t = 0; t < T; ++t) keys += hm.pos[t] + 1;
      // keys and values of 64 or 128 numbers, bfloat16: the tcgen05 prompt kernel and the TMA-staged decode kernels of the
      // Llama family (every head its own key/value head); everything else: the mma.sync / per-row kernels
      const bool tc = !e->f32 && (h.dim == 64 || h.dim == 128) && h.vdim == h.dim && ldq % 8 == 0 && (bs & (bs - 1)) == 0 && ((uintptr_t)q & 15) == 0 &&
                      (!decode_only || (e->ws_attn && paged_attn_extras_decode_ok(B, H, H, h.dim, bs)));
      const int max_seq_bound = decode_only ? max_blocks * bs : 0;
      HFWD(decode_only ? C_ATT_DEC : C_ATT_GEN, (decode_only ? keys : (double)T) * H * (h.dim + h.vdim) * es + (double)T * H * (h.dim + h.vdim) * es,
           2.0 * keys * H * (h.dim + h.vdim),
           tc ? paged_attn_extras(e->mixbuf, q, ldq, L.kc, L.vc, m.btab, max_blocks, m.seq_lens, m.qsl, B, T, aa.max_q, std::max(max_seq_bound, 1), H, H, h.dim, bs,
                                  h.scale, 0.f, nullptr, e->ws_attn, e->ws_attn_bytes, st)
              : attn_bias_chunk(aa, st));
      if (h.out_gate) HFWD(C_ACT, (double)T * nv * 3 * es, 0, sigmoid_gate_mul(e->mixbuf, nv, at(e->pbuf, L.lat_g), ldp, T, nv, elt, st));
      DENSE(e->obuf1, d, e->mixbuf, nv, L.o, T, ACT_NONE);
      add_src(e->obuf1, d, 1.f);
    } else {
      const int ka = h.heads * h.vdim, ko = L.o2.K, ldp = L.proj.N;
      DENSE(e->pbuf, ldp, e->hx, d, L.proj, T, ACT_NONE);
      {
        LinearArgs a;      // gate pre-activations of the matrix memory stay in fp32
        a.x = e->hx; a.ldx = d; a.w = L.gates.w; a.bias = L.gates.b; a.y = e->gates32; a.ldy = 2 * h.m_heads; a.T = T; a.N = 2 * h.m_heads; a.K = d;
        a.elt = elt; a.out_f32 = true;
        HFWD(C_MLSTM, Td * es, 4.0 * Td * h.m_heads, linear_any(a, st));
      }
      HFWD(C_KVW, 2.0 * T * h.kv_heads * (h.dim + h.vdim) * es, 0,
           kv_write_any(at(e->pbuf, L.off_k), ldp, at(e->pbuf, L.off_v), ldp, m.slots, L.kc, L.vc, T, h.kv_heads, h.dim, h.vdim, bs, elt, st));
      AttnBiasArgs aa;
      aa.q = e->pbuf; aa.ldq = ldp; aa.out = e->mixbuf; aa.ldo = ko; aa.k_cache = L.kc; aa.v_cache = L.vc;
      aa.block_table = m.btab; aa.max_blocks = max_blocks; aa.seq_lens = m.seq_lens; aa.qsl = m.qsl; aa.positions = m.pos; aa.token_req = m.treq;
      aa.B = B; aa.T = T; aa.H = h.heads; aa.G = h.kv_heads; aa.dim = h.dim; aa.vdim = h.vdim; aa.block_size = bs; aa.chunk = h.chunk;
      aa.scale = h.scale; aa.bias_span = 8.f; aa.out_scale = h.left_scale; aa.elt = elt;
      for (int r = 0; r < B; ++r) aa.max_q = std::max(aa.max_q, hm.qsl[r + 1] - hm.qsl[r]);
      while (aa.num_decode < B && hm.qsl[aa.num_decode + 1] - hm.qsl[aa.num_decode] == 1) ++aa.num_decode;
      double keys = 0;                                   // visible keys over all rows
      for (int t = 0; t < T; ++t) keys += h.chunk > 0 ? hm.pos[t] % h.chunk + 1 : hm.pos[t] + 1;
      HFWD(decode_only ? C_ATT_DEC : C_ATT_GEN, (decode_only ? keys : (double)T) * h.kv_heads * (h.dim + h.vdim) * es + (double)T * h.heads * (h.dim + h.vdim) * es,
           2.0 * keys * h.heads * (h.dim + h.vdim), attn_bias_chunk(aa, st));
      MlstmArgs ma;
      ma.q = at(e->pbuf, L.off_mq); ma.k = at(e->pbuf, L.off_mk); ma.v = at(e->pbuf, L.off_mv); ma.g = at(e->pbuf, L.off_mg); ma.ld = ldp;
      ma.gates = e->gates32; ma.o_scratch = e->mo32; ma.norm_w = L.m_norm; ma.out = at(e->mixbuf, ka); ma.ldo = ko;
      ma.state = e->state + L.state_off; ma.slot_stride = e->slot_stride; ma.slots = m.sslot; ma.qsl = m.qsl; ma.positions = m.pos;
      ma.B = B; ma.T = T; ma.H = h.m_heads; ma.dim = h.m_dim; ma.vdim = h.m_vdim;
      ma.cap = h.gate_cap; ma.q_scale = 1.f / sqrtf((float)h.m_dim); ma.eps = s.eps; ma.den_eps = 1e-6f; ma.out_scale = h.right_scale; ma.elt = elt;
      HFWD(C_MLSTM, 2.0 * B * mlstm_state_floats(h.m_heads, h.m_dim, h.m_vdim) * 4 + (double)T * h.m_heads * (2 * h.m_dim + 3 * h.m_vdim) * es,
           4.0 * T * h.m_heads * (double)h.m_dim * h.m_vdim, mlstm_step(ma, st));
      DENSE(e->obuf1, d, e->mixbuf, ko, L.o2, T, ACT_NONE);
      add_src(e->obuf1, d, 1.f);
    }
    if (s.hyb_prenorm_pair && h.mlp != HybridLayerSpec::NONE) {
      // the feed-forward reads a norm of the stream that already holds the mixer's output
      { const double nsrc = cb.n + (s.hyb_postnorm ? 1 : 0); HFWD(C_ACT, Td * (8.0 * S + nsrc * es), 0, flush()); }      // post-norm models also write the next normed row
      sub = 1;
      if (!hyper && !s.hyb_postnorm) HFWD(C_NORM, Td * (4 + es), 0, layer_norm(e->hx, nullptr, L.norm2, T, 1.f));
    }
    if (h.mlp == HybridLayerSpec::DENSE && h.ff_silu_bias) {
      // silu(gate h + b) * (up h + b): one product over [gate | up] with the biases, the pair formed from its rows
      const int f = h.ff;
      void* act = at(e->ffbuf, (int64_t)2 * f * T);
      if (!e->f32 && f % 64 == 0 && d % 8 == 0) {
        // [T, 2f] never reaches memory: biases and the gated pair in the epilogue of the tensor-core GEMM
        HFWD(T <= 256 ? C_GEMM_S : C_GEMM_L, es * (2.0 * f * d + (double)T * (d + f)), 4.0 * T * (double)f * d,
             gemm_silu_gate_bias(act, e->hx, L.ff_gate, L.ff_gate_b, T, f, d, st));
      } else {
        DENSE(e->ffbuf, 2 * f, e->hx, d, L.up, T, ACT_NONE);
        HFWD(C_ACT, (double)T * f * 3 * es, 0, silu_mul_halves(act, e->ffbuf, T, f, elt, st));
      }
      DENSE(e->obuf2, d, act, f, L.down, T, ACT_NONE);
      add_src(e->obuf2, d, 1.f);
    } else if (h.mlp == HybridLayerSpec::DENSE && h.ff_limit > 0.f) {
      // clamped gated unit: bfloat16 forms the pair in the epilogue of the tensor-core GEMM over [gate | up]
      const int f = h.ff;
      const double gb = es * (2.0 * f * d + (double)T * (d + f)), gf = 4.0 * T * (double)f * d;
      if (!e->f32 && f % 64 == 0 && d % 8 == 0) {
        HFWD(T <= 256 ? C_GEMM_S : C_GEMM_L, gb, gf, kge_gemm_clamped_glu_bf16(e->ffbuf, e->hx, L.ff_gate, T, f, d, 1.702f, h.ff_limit, nullptr, 0, st));
      } else {
        LinearArgs sg;
        sg.x = e->hx; sg.ldx = d; sg.w = L.ff_gate; sg.w2 = L.up.w; sg.y = e->ffbuf; sg.ldy = f; sg.T = T; sg.N = f; sg.K = d;
        sg.glu = GLU_CLAMPED_SIGMOID; sg.glu_limit = h.ff_limit; sg.elt = elt; sg.out_f32 = e->f32;
        HFWD(T <= 256 ? C_GEMM_S : C_GEMM_L, gb, gf, linear_any(sg, st));
      }
      DENSE(e->obuf2, d, e->ffbuf, f, L.down, T, ACT_NONE);
      add_src(e->obuf2, d, 1.f);
    } else if (h.mlp == HybridLayerSpec::DENSE) {
      DENSE(e->ffbuf, h.ff, e->hx, d, L.up, T, ACT_GELU_ERF);
      DENSE(e->obuf2, d, e->ffbuf, h.ff, L.down, T, ACT_NONE);
      add_src(e->obuf2, d, 1.f);
    } else if (h.mlp == HybridLayerSpec::MOE) {
      MoeRouteArgs ra;
      ra.h = e->hx; ra.ldh = d; ra.w_router = L.router.w; ra.b_router = L.router_b; ra.T = T; ra.d = d; ra.E = h.experts; ra.top = h.top;
      const bool w_out = h.route != HybridLayerSpec::ROUTE_SIGMOID_IN;      // the routing weight multiplies the expert's output (in the fp32 sum below)
      const bool clamped = h.glu == HybridLayerSpec::GLU_CLAMPED;
      const bool ungated = h.glu == HybridLayerSpec::GLU_NONE_RELU2;      // one front matrix per expert, relu(.)^2
      ra.score_fn = h.route == HybridLayerSpec::ROUTE_SOFTMAX_TOP ? 2 : h.route == HybridLayerSpec::ROUTE_SOFTMAX_ALL ? 1 : 0; ra.renorm = false;
      ra.weight_scale = h.router_scale;
      if (L.s_sg) { ra.w_extra = L.s_sg; ra.extra_sigmoid = e->gates32; }      // the shared expert's per-token gate rides along, kept in fp32
      ra.group_off = e->moe_goff; ra.perm_token = e->moe_ptok; ra.perm_weight = e->moe_pw; ra.perm_dest = e->moe_pdest;
      ra.choice_expert = e->moe_cexp; ra.choice_weight = e->moe_cw; ra.elt = elt;
      const int np = T * h.top;
      // bfloat16 prompt steps with enough routed rows: groups padded to 256 rows for the grouped tensor-core GEMMs
      const int np_pad = (np / 256 + h.experts + 1) * 256;
      const bool grouped = !e->f32 && !decode_only && np >= 512 && h.expert_ff % 64 == 0 && d % 8 == 0 && e->moe_xperm && np_pad <= e->moe_rows_padded;
      if (grouped) { ra.pad = 256; ra.rows_padded = np_pad; ra.tile_group = e->moe_tile_group; }
      HFWD(C_MOE, Td * es + (double)h.experts * d * es, 2.0 * Td * h.experts, moe_route(ra, st));
      ++e->launches;
      const double wexp = (double)std::min(h.experts, np) * h.expert_ff * d * es;      // weights of the experts that are touched (at most)
      if (grouped) {
        // prompt steps: every expert's routed rows, padded to a multiple of 256, are contiguous; ONE tensor-core launch
        // runs the gated front half of all experts (the pair formed in the epilogue) and one the down projections; each
        // 256-row tile takes its expert's weights from the stacked tensors.  Nothing comes back to the host.
        const int eff = h.expert_ff;
        HFWD(C_MOE, (double)np_pad * d * 4, 0, moe_gather_rows(e->moe_xperm, e->hx, d, e->moe_ptok, w_out ? nullptr : e->moe_pw, np_pad, d, st));
        HFWD(C_MOE, 2.0 * ((ungated ? 1.0 : 2.0) * h.experts * eff * d + (double)np_pad * (d + eff)), (ungated ? 2.0 : 4.0) * np * (double)eff * d,
             gemm_grouped(e->moe_hidden, e->moe_xperm, L.e_gate, np_pad, eff, d, h.experts, e->moe_tile_group, ungated ? -2 : clamped ? 1 : 0, 1.702f, h.expert_limit, st));
        HFWD(C_MOE, 2.0 * ((double)h.experts * eff * d + (double)np_pad * (d + eff)), 2.0 * np * (double)eff * d,
             gemm_grouped(e->moe_operm, e->moe_hidden, L.e_down, np_pad, d, eff, h.experts, e->moe_tile_group, -1, 0.f, 0.f, st));
        HFWD(C_MOE, (double)np * d * 4, 0, moe_scatter_rows(e->moe_out, e->moe_operm, e->moe_pdest, np_pad, d, st));
      } else {
      LinearArgs g;      // experts' gated front half on the gathered, weighted rows
      g.x = e->hx; g.ldx = d; g.w = L.e_gate; g.w2 = L.e_up; g.y = e->moe_hidden; g.ldy = h.expert_ff; g.T = np; g.N = h.expert_ff; g.K = d;
      g.nz = h.experts; g.w_zs = (int64_t)2 * h.expert_ff * d; g.group_off = e->moe_goff; g.max_rows = np; g.xrows = e->moe_ptok; g.row_scale = w_out ? nullptr : e->moe_pw;
      if (clamped) { g.glu = GLU_CLAMPED_SIGMOID; g.glu_limit = h.expert_limit; }
      if (ungated) { g.w2 = nullptr; g.w_zs = (int64_t)h.expert_ff * d; g.act = ACT_RELU2; }
      g.elt = elt; g.out_f32 = e->f32;
      HFWD(C_MOE, (ungated ? 1 : 2) * wexp + (double)np * (d + h.expert_ff) * es, (ungated ? 2.0 : 4.0) * np * (double)h.expert_ff * d, linear_any(g, st));
      LinearArgs dn;     // experts' down projection, scattered to row (token * top + choice)
      dn.x = e->moe_hidden; dn.ldx = h.expert_ff; dn.w = L.e_down; dn.y = e->moe_out; dn.ldy = d; dn.T = np; dn.N = d; dn.K = h.expert_ff;
      dn.nz = h.experts; dn.w_zs = (int64_t)d * h.expert_ff; dn.group_off = e->moe_goff; dn.max_rows = np; dn.yrows = e->moe_pdest;
      dn.elt = elt; dn.out_f32 = e->f32;
      HFWD(C_MOE, wexp + (double)np * (d + h.expert_ff) * es, 2.0 * np * (double)h.expert_ff * d, linear_any(dn, st));
      }
      if (h.shared_ff > 0) {
        const int f = h.shared_ff;
        const double gb = es * (2.0 * f * d + (double)T * (d + f)), gf = 4.0 * T * (double)f * d;
        if (!e->f32 && f % 64 == 0 && d % 8 == 0) {
          // [T, 2f] never reaches memory: the gated pair is formed in the epilogue of the tensor-core GEMM
          HFWD(T <= 256 ? C_GEMM_S : C_GEMM_L, gb, gf,
               clamped ? kge_gemm_clamped_glu_bf16(e->ffbuf, e->hx, L.s_gate.w, T, f, d, 1.702f, h.shared_limit, nullptr, 0, st)
                       : kge_gemm_silu_gate_ws_bf16(e->ffbuf, e->hx, L.s_gate.w, T, f, d, nullptr, 0, st));
        } else {
          LinearArgs sg;
          sg.x = e->hx; sg.ldx = d; sg.w = L.s_gate.w; sg.w2 = L.s_up.w; sg.y = e->ffbuf; sg.ldy = f; sg.T = T; sg.N = f; sg.K = d;
          if (clamped) { sg.glu = GLU_CLAMPED_SIGMOID; sg.glu_limit = h.shared_limit; }
          sg.elt = elt; sg.out_f32 = e->f32;
          HFWD(T <= 256 ? C_GEMM_S : C_GEMM_L, gb, gf, linear_any(sg, st));
        }
        DENSE(e->obuf2, d, e->ffbuf, f, L.s_down, T, ACT_NONE);
      }
      // sum in a fixed order: mixer, the token's experts by choice, the shared expert
      for (int k = 0; k < h.top; ++k) {
        if (cb.n == 4) HFWD(C_ACT, Td * (8 + 4 * es), 0, flush_more());
        add_src(at(e->moe_out, (int64_t)k * d), h.top * d, 1.f, w_out ? e->moe_cw + k : nullptr, h.top);
      }
      if (h.shared_ff > 0) { if (cb.n == 4) HFWD(C_ACT, Td * (8 + 4 * es), 0, flush_more()); add_src(e->obuf2, d, 1.f, L.s_sg ? e->gates32 : nullptr, 1); }
    }
    { const double nsrc = cb.n + (s.hyb_postnorm ? 1 : 0); HFWD(C_ACT, Td * (8.0 * S + nsrc * es), 0, flush()); }      // post-norm models also write the next normed row
    if (e->layer_dump_host && (int64_t)(i + 1) * T * d <= e->layer_dump_cap) {
      if (hyper) { if (int rc = stream_read(nullptr, nullptr, nullptr, nullptr, T, 1.f, e->y32)) return rc; }      // the sum of the streams
      KGE_CUDA_OK(cudaMemcpyAsync(e->layer_dump_host + (int64_t)i * T * d, hyper ? e->y32 : e->res32, (size_t)T * d * 4, cudaMemcpyDeviceToHost, st));
      KGE_CUDA_OK(cudaStreamSynchronize(st));
    }
  }
  if (R > 0) {
    const int Rm = e->cfg.max_num_seqs;
    KGE_REQUIRE(R <= std::max(Rm, e->cfg.max_num_batched_tokens), "hybrid_forward: %d logits rows", R);
    const double hb = es * ((double)s.vocab * d + (double)R * (d + s.vocab)), hf = 2.0 * R * (double)s.vocab * d;
    if (e->hyb_head_tc) {
      // norm (the logits' multiplier folded into it), then the tensor-core GEMM straight into the 16-bit logits
      if (hyper) HFWD(C_NORM, (double)R * d * (4.0 * S + es), 0, stream_read(e->hsel, nullptr, m.rows, e->final_w, R, s.logit_scale, nullptr));
      else HFWD(C_NORM, (double)R * d * (4 + es), 0, layer_norm(e->hsel, m.rows, e->final_w, R, s.logit_scale));
      HFWD(R <= 256 ? C_GEMM_S : C_GEMM_L, hb, hf, kge_gemm_bf16(e->logits, e->hsel, e->lm_head, nullptr, R, s.vocab, d, 0, nullptr, 0, st));
      if (s.logit_softcap > 0.f) HFWD(C_SAMPLE, (double)R * s.vocab * (e->want_logits32 ? 8 : 4), 0, softcap_rows(e->want_logits32 ? e->logits32 : nullptr, e->logits, R, s.vocab, e->ld_logits, s.logit_softcap, st));
      else if (e->want_logits32) HFWD(C_SAMPLE, (double)R * s.vocab * 6, 0, elt16_to_f32(e->logits32, e->logits, (int64_t)R * s.vocab, st));
    } else {
      if (hyper) HFWD(C_NORM, (double)R * d * (4.0 * S + es), 0, stream_read(e->hsel, nullptr, m.rows, e->final_w, R, 1.f, nullptr));
      else HFWD(C_NORM, (double)R * d * (4 + es), 0, layer_norm(e->hsel, m.rows, e->final_w, R, 1.f));
      LinearArgs a;
      a.x = e->hsel; a.ldx = d; a.w = e->lm_head; a.y = e->logits32; a.ldy = s.vocab; a.T = R; a.N = s.vocab; a.K = d;
      a.alpha = s.logit_scale; a.elt = elt; a.out_f32 = true;
      HFWD(R <= 256 ? C_GEMM_S : C_GEMM_L, hb, hf, linear_any(a, st));
      if (s.logit_softcap > 0.f) HFWD(C_SAMPLE, (double)R * s.vocab * 8, 0, softcap_rows(e->logits32, nullptr, R, s.vocab, 0, s.logit_softcap, st));
      // the samplers read 16-bit logits, rows padded to the 16-byte alignment they ask for
      if (R <= Rm) HFWD(C_SAMPLE, (double)R * s.vocab * 6, 0, logits_to_elt16(e->logits, e->logits32, R, s.vocab, e->ld_logits, false, st));
    }
    if (R <= Rm) {
      if (int rc = mask_step_logits(e)) return rc;
      if (any_random) HFWD(C_SAMPLE, (double)R * s.vocab * 2, 0, kge_sample(e->d_out, e->logits, R, s.vocab, e->ld_logits, m.temp, m.top_k, m.top_p, nullptr, m.seeds, 0, nullptr, 0, st));
      else HFWD(C_SAMPLE, (double)R * s.vocab * 2, 0, kge_argmax(e->d_out, e->logits, R, s.vocab, e->ld_logits, st));
    }
  }
  return 0;
}

}  // namespace kge
