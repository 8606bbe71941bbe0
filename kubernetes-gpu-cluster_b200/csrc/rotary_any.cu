// Rotary positions for layer-list models: partial (the first rot_dims dimensions of a head), interleaved pairs, plain
// or YaRN-scaled frequencies; fused with what surrounds the rotation in an attention mixer - an RMS norm over the whole
// q and k projections, the write of the rotated keys into the paged cache, and the write of the values (a projection of
// their own, or the un-normed, un-rotated key projection).  One block per token: sums of squares in fp32, the token's
// cos / sin pairs once in shared memory (angle = position * frequency formed in double precision, so long contexts
// lose nothing: whole turns are removed in double, the remainder goes through the fp32 sine and cosine), then every head reads them.
#include <math.h>

#include <algorithm>

#include "common.cuh"
#include "elt_access.cuh"
#include "hybrid_ops.h"

namespace kge {

void rotary_frequencies(int dims, double base, double factor, double original, double fast, double slow, double* freq, float* mult) {
  const int half = dims / 2;
  for (int i = 0; i < half; ++i) freq[i] = pow(base, -2.0 * i / dims);
  *mult = 1.f;
  if (factor > 0.0) {
    const double pi = 3.14159265358979323846;
    auto corr = [&](double turns) { return dims * log(original / (2.0 * pi * turns)) / (2.0 * log(base)); };
    const double lo = std::max(floor(corr(fast)), 0.0), hi = std::min(ceil(corr(slow)), (double)(dims - 1));
    for (int i = 0; i < half; ++i) {
      const double ramp = std::min(std::max((i - lo) / std::max(hi - lo, 0.001), 0.0), 1.0);
      freq[i] = freq[i] / factor * ramp + freq[i] * (1.0 - ramp);
    }
    *mult = (float)(0.1 * log(factor) + 1.0);
  }
}

// sin and cos of an angle formed in double precision: whole turns are taken off in double (three operations), the rest -
// within [-pi, pi], exact to an fp32 rounding - goes through the fp32 functions
__device__ __forceinline__ void sincos_reduced(double ang, float* s, float* c) {
  const double turns = rint(ang * 0.15915494309189535);
  sincosf((float)fma(-turns, 6.283185307179586, ang), s, c);
}

template <typename E>
__global__ void __launch_bounds__(256) rotary_norm_kvwrite_kernel(RotaryArgs a) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ float cs[];                 // [rot_dims / 2] cos, then sin (multiplier applied)
  __shared__ float red[33];
  const int t = blockIdx.x, half = a.rot_dims >> 1, nq = a.H * a.dim, nk = a.G * a.dim;
  const int pos = a.positions[t];
  for (int i = threadIdx.x; i < half; i += blockDim.x) {
    float s, c;
    sincos_reduced((double)pos * a.freq[i], &s, &c);
    cs[i] = c * a.mult;
    cs[half + i] = s * a.mult;
  }
  E* q = (E*)a.q + (int64_t)t * a.ldq;
  const E* k = (const E*)a.k + (int64_t)t * a.ldk;
  float inv_q = 1.f, inv_k = 1.f;
  if (a.q_norm_w) {
    float ss = 0.f;
    for (int c = threadIdx.x; c < nq; c += blockDim.x) { const float v = ldf(q + c); ss = fmaf(v, v, ss); }
    inv_q = 1.f / sqrtf(block_sum(ss, red) / (float)nq + a.eps);
    __syncthreads();
  }
  if (a.k_norm_w) {
    float ss = 0.f;
    for (int c = threadIdx.x; c < nk; c += blockDim.x) { const float v = ldf(k + c); ss = fmaf(v, v, ss); }
    inv_k = 1.f / sqrtf(block_sum(ss, red) / (float)nk + a.eps);
  }
  __syncthreads();
  const int64_t slot = a.slots ? a.slots[t] : -1;
  const int64_t blk = slot >= 0 ? slot / a.block_size : 0, off = slot >= 0 ? slot % a.block_size : 0;
  // values first: they may be the key projection as it came in
  if (slot >= 0 && a.v_cache) {
    const E* v = a.v ? (const E*)a.v + (int64_t)t * a.ldv : k;
    E* vc = (E*)a.v_cache;
    for (int c = threadIdx.x; c < a.G * a.vdim; c += blockDim.x) {
      const int g = c / a.vdim, d = c % a.vdim;
      vc[((blk * a.G + g) * a.block_size + off) * a.vdim + d] = v[c];
    }
  }
  // one item = one pair of neighbouring dimensions of one head (dim even), or the single last dimension of an odd head size
  const int ppd = (a.dim + 1) >> 1;
  for (int idx = threadIdx.x; idx < (a.H + a.G) * ppd; idx += blockDim.x) {
    const int hh = idx / ppd, pi = idx % ppd, d0 = 2 * pi;
    const bool isq = hh < a.H;
    const int head = isq ? hh : hh - a.H, col = head * a.dim + d0;
    const bool two = d0 + 1 < a.dim;
    const E* src = isq ? q : k;
    const E* nw = (const E*)(isq ? a.q_norm_w : a.k_norm_w);
    const float inv = isq ? inv_q : inv_k;
    float u = ldf(src + col) * inv, v = two ? ldf(src + col + 1) * inv : 0.f;
    if (nw) { u *= ldf(nw + col); if (two) v *= ldf(nw + col + 1); }
    if (d0 + 1 < a.rot_dims) {
      const float c = cs[pi], s = cs[half + pi];
      const float ru = u * c - v * s, rv = v * c + u * s;
      u = ru; v = rv;
    }
    if (isq) {
      stf(q + col, u); if (two) stf(q + col + 1, v);
    } else if (slot >= 0 && a.k_cache) {
      E* kc = (E*)a.k_cache + ((blk * a.G + head) * a.block_size + off) * a.dim + d0;
      stf(kc, u); if (two) stf(kc + 1, v);
    }
  }
}

// bfloat16, head size a multiple of 8, 16-byte aligned rows and caches: a token's q and k rows are read ONCE, eight values
// (16 bytes) per piece, and stay in registers for the sums of squares and for norm, rotation and the stores (16 bytes each).
// Up to RV_MAX pieces per thread: (H + G) * dim <= 256 * 8 * RV_MAX.
constexpr int RV_MAX = 4;
__global__ void __launch_bounds__(256) rotary_norm_kvwrite_vec_kernel(RotaryArgs a) {
  pdl_launch_dependents();
  pdl_wait();
  typedef __nv_bfloat16 E;
  extern __shared__ float cs[];                 // [rot_dims / 2] cos, then sin (multiplier applied)
  __shared__ float red[33];
  const int t = blockIdx.x, half = a.rot_dims >> 1, nq = a.H * a.dim, nk = a.G * a.dim, pq = nq >> 3, pall = (nq + nk) >> 3;
  const int pos = a.positions[t];
  E* q = (E*)a.q + (int64_t)t * a.ldq;
  const E* k = (const E*)a.k + (int64_t)t * a.ldk;
  uint4 raw[RV_MAX], wraw[RV_MAX];              // the norm weights travel with the rows: one memory round trip, not two
  float ssq = 0.f, ssk = 0.f;
  const int64_t slot = a.slots ? a.slots[t] : -1;
#pragma unroll
  for (int i = 0; i < RV_MAX; ++i) {
    const int p = threadIdx.x + i * 256;
    raw[i] = wraw[i] = make_uint4(0u, 0u, 0u, 0u);
    if (p < pall) {
      raw[i] = p < pq ? *reinterpret_cast<const uint4*>(q + 8 * p) : *reinterpret_cast<const uint4*>(k + 8 * (p - pq));
      const E* nw0 = (const E*)(p < pq ? a.q_norm_w : a.k_norm_w);
      if (nw0) wraw[i] = *reinterpret_cast<const uint4*>(nw0 + (p < pq ? 8 * p : 8 * (p - pq)));
      const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raw[i]);
      float ss = 0.f;
#pragma unroll
      for (int j = 0; j < 4; ++j) { const float2 f = __bfloat1622float2(h2[j]); ss = fmaf(f.x, f.x, ss); ss = fmaf(f.y, f.y, ss); }
      if (p < pq) ssq += ss; else ssk += ss;
    }
  }
  // the token's cos / sin pairs, while the rows are on their way
  for (int i = threadIdx.x; i < half; i += blockDim.x) {
    float s, c;
    sincos_reduced((double)pos * a.freq[i], &s, &c);
    cs[i] = c * a.mult;
    cs[half + i] = s * a.mult;
  }
  // both sums of squares in one pass over the block
  float inv_q = 1.f, inv_k = 1.f;
  {
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    ssq = warp_sum(ssq); ssk = warp_sum(ssk);
    if (lane == 0) { red[wid] = ssq; red[8 + wid] = ssk; }
    __syncthreads();
    float tq = lane < 8 ? red[lane] : 0.f, tk = lane < 8 ? red[8 + lane] : 0.f;
    tq = warp_sum(tq); tk = warp_sum(tk);
    if (a.q_norm_w) inv_q = 1.f / sqrtf(tq / (float)nq + a.eps);
    if (a.k_norm_w) inv_k = 1.f / sqrtf(tk / (float)nk + a.eps);
  }
  const int64_t blk = slot >= 0 ? slot / a.block_size : 0, off = slot >= 0 ? slot % a.block_size : 0;
#pragma unroll
  for (int i = 0; i < RV_MAX; ++i) {
    const int p = threadIdx.x + i * 256;
    if (p >= pall) continue;
    const bool isq = p < pq;
    const int col = isq ? 8 * p : 8 * (p - pq), head = col / a.dim, d0 = col % a.dim;
    const int64_t cache_off = ((blk * a.G + head) * a.block_size + off) * a.dim + d0;
    if (!isq && slot >= 0 && a.v_cache && !a.v) *reinterpret_cast<uint4*>((E*)a.v_cache + cache_off) = raw[i];     // values = the raw key projection
    const E* nw = (const E*)(isq ? a.q_norm_w : a.k_norm_w);
    const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raw[i]);
    const __nv_bfloat162* w2 = reinterpret_cast<const __nv_bfloat162*>(&wraw[i]);
    const float inv = isq ? inv_q : inv_k;
    uint4 outv;
    __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&outv);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float2 f = __bfloat1622float2(h2[j]);
      f.x *= inv; f.y *= inv;
      if (nw) { const float2 g = __bfloat1622float2(w2[j]); f.x *= g.x; f.y *= g.y; }
      const int d = d0 + 2 * j;
      if (d + 1 < a.rot_dims) {
        const float c = cs[d >> 1], s = cs[half + (d >> 1)];
        const float ru = f.x * c - f.y * s, rv = f.y * c + f.x * s;
        f.x = ru; f.y = rv;
      }
      o2[j] = __floats2bfloat162_rn(f.x, f.y);
    }
    if (isq) *reinterpret_cast<uint4*>(q + col) = outv;
    else if (slot >= 0 && a.k_cache) *reinterpret_cast<uint4*>((E*)a.k_cache + cache_off) = outv;
  }
  // a value projection of its own
  if (slot >= 0 && a.v_cache && a.v) {
    const E* v = (const E*)a.v + (int64_t)t * a.ldv;
    E* vc = (E*)a.v_cache;
    for (int c = threadIdx.x; c < a.G * a.vdim; c += blockDim.x) {
      const int g = c / a.vdim, d = c % a.vdim;
      vc[((blk * a.G + g) * a.block_size + off) * a.vdim + d] = v[c];
    }
  }
}

int rotary_norm_kvwrite(const RotaryArgs& a, cudaStream_t st) {
  if (a.T <= 0) return 0;
  KGE_REQUIRE(a.q && a.k && a.positions && a.H > 0 && a.G > 0 && a.dim > 0 && a.rot_dims >= 0 && a.rot_dims <= a.dim && a.rot_dims % 2 == 0 &&
              (a.rot_dims == 0 || a.freq), "rotary_norm_kvwrite: bad arguments");
  KGE_REQUIRE(a.v || a.vdim == a.dim, "rotary_norm_kvwrite: values taken from the keys need vdim = dim");
  const size_t smem = (size_t)std::max(a.rot_dims, 2) * 4;
  auto al16 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
  if (a.elt == KGE_ELT_BF16 && a.dim % 8 == 0 && a.ldq % 8 == 0 && a.ldk % 8 == 0 && (a.H + a.G) * a.dim <= 256 * 8 * RV_MAX && al16(a.q) && al16(a.k) &&
      al16(a.k_cache) && al16(a.v_cache) && al16(a.q_norm_w) && al16(a.k_norm_w) && (a.v || a.vdim == a.dim)) {
    KGE_CUDA_OK(launch_pdl(rotary_norm_kvwrite_vec_kernel, dim3(a.T), dim3(256), smem, st, a));
    return 0;
  }
  cudaError_t ce = a.elt == KGE_ELT_F32 ? launch_pdl(rotary_norm_kvwrite_kernel<float>, dim3(a.T), dim3(256), smem, st, a)
                                        : launch_pdl(rotary_norm_kvwrite_kernel<__nv_bfloat16>, dim3(a.T), dim3(256), smem, st, a);
  KGE_CUDA_OK(ce);
  return 0;
}

// ---------------------------------------------------------------------------------------------------------------
// Norms per head and rotation in halves.  One block per token, one warp per head in turn (q heads, then key heads, then
// value heads): the warp sums the head's squares (fp32), then walks the head's pairs (i, i + rot_dims / 2); dimensions
// beyond rot_dims pass with the norm only.  Values turn over their whole width by the token's own position.  The token's
// cos / sin tables (rot_dims / 2 entries for q and k, vdim / 2 for the values) are formed once per block.
template <typename E>
__global__ void __launch_bounds__(256) head_norm_rotary_kvwrite_kernel(HeadRotaryArgs a) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ float hcs[];                // [half] cos, [half] sin, [vhalf] cos, [vhalf] sin
  const int t = blockIdx.x, half = a.rot_dims >> 1, vhalf = a.v_freq ? a.vdim >> 1 : 0;
  float *qc = hcs, *qs = hcs + half, *vcs = hcs + 2 * half, *vsn = vcs + vhalf;
  const int pos = a.positions[t];
  for (int i = threadIdx.x; i < half + vhalf; i += blockDim.x) {
    float s, c;
    if (i < half) { sincos_reduced((double)pos * a.freq[i], &s, &c); qc[i] = c; qs[i] = s; }
    else { sincos_reduced((double)pos * a.v_freq[i - half], &s, &c); vcs[i - half] = c; vsn[i - half] = s; }
  }
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  const int64_t slot = a.slots ? a.slots[t] : -1;
  const int64_t blk = slot >= 0 ? slot / a.block_size : 0, off = slot >= 0 ? slot % a.block_size : 0;
  const int heads = a.H + a.G + (a.v ? a.G : 0);
  for (int hh = warp; hh < heads; hh += nw) {
    if (hh < a.H + a.G) {
      const bool isq = hh < a.H;
      const int h = isq ? hh : hh - a.H;
      const E* src = isq ? (const E*)a.q + (int64_t)t * a.ldq + h * a.dim : (const E*)a.k + (int64_t)t * a.ldk + h * a.dim;
      const bool norm = isq ? a.norm_q : a.norm_k;
      const E* w = (const E*)(isq ? a.q_norm_w : a.k_norm_w);
      float inv = 1.f;
      if (norm) {
        float ss = 0.f;
        for (int c = lane; c < a.dim; c += 32) { const float v = ldf(src + c); ss = fmaf(v, v, ss); }
        inv = 1.f / sqrtf(warp_sum(ss) / (float)a.dim + a.eps);
      }
      E* dst = nullptr;
      if (isq) dst = (E*)a.q + (int64_t)t * a.ldq + h * a.dim;
      else if (slot >= 0) dst = (E*)a.k_cache + ((blk * a.G + h) * a.block_size + off) * a.dim;
      if (!dst) continue;
      // every lane reads both numbers of its pairs before it writes them (q is rewritten in place)
      for (int i = lane; i < half; i += 32) {
        const float u = ldf(src + i) * inv * (w ? ldf(w + i) : 1.f), v = ldf(src + half + i) * inv * (w ? ldf(w + half + i) : 1.f);
        stf(dst + i, u * qc[i] - v * qs[i]);
        stf(dst + half + i, v * qc[i] + u * qs[i]);
      }
      for (int c = 2 * half + lane; c < a.dim; c += 32) stf(dst + c, ldf(src + c) * inv * (w ? ldf(w + c) : 1.f));
    } else if (slot >= 0) {
      const int g = hh - a.H - a.G;
      const E* src = (const E*)a.v + (int64_t)t * a.ldv + g * a.vdim;
      E* dst = (E*)a.v_cache + ((blk * a.G + g) * a.block_size + off) * a.vdim;
      if (a.v_freq) {
        for (int i = lane; i < vhalf; i += 32) {
          const float u = ldf(src + i), v = ldf(src + vhalf + i);
          stf(dst + i, u * vcs[i] - v * vsn[i]);
          stf(dst + vhalf + i, v * vcs[i] + u * vsn[i]);
        }
      } else {
        for (int c = lane; c < a.vdim; c += 32) dst[c] = src[c];
      }
    }
  }
}

int head_norm_rotary_kvwrite(const HeadRotaryArgs& a, cudaStream_t st) {
  if (a.T <= 0) return 0;
  KGE_REQUIRE(a.rot_dims >= 0 && a.rot_dims % 2 == 0 && a.rot_dims <= a.dim && (a.rot_dims == 0 || a.freq) && (!a.v_freq || a.vdim % 2 == 0),
              "head_norm_rotary_kvwrite: %d of %d dimensions turn (values: %d)", a.rot_dims, a.dim, a.vdim);
  const size_t smem = (size_t)(a.rot_dims + (a.v_freq ? a.vdim : 0)) * 4;
  cudaError_t ce = a.elt == KGE_ELT_F32 ? launch_pdl(head_norm_rotary_kvwrite_kernel<float>, dim3(a.T), dim3(256), smem, st, a)
                                        : launch_pdl(head_norm_rotary_kvwrite_kernel<__nv_bfloat16>, dim3(a.T), dim3(256), smem, st, a);
  KGE_CUDA_OK(ce);
  return 0;
}

// one block per token, one warp per head in turn
template <typename E>
__global__ void __launch_bounds__(256) rotate_heads_halves_kernel(E* x, int ldx, const int32_t* positions, const double* freq, int H, int n, float sign) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ float rcs[];                // [n / 2] cos, then sin
  const int t = blockIdx.x, half = n >> 1;
  const int pos = positions[t];
  for (int i = threadIdx.x; i < half; i += blockDim.x) {
    float s, c;
    sincos_reduced((double)pos * freq[i], &s, &c);
    rcs[i] = c; rcs[half + i] = sign * s;
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < H * half; idx += blockDim.x) {
    const int h = idx / half, i = idx % half;
    E* p = x + (int64_t)t * ldx + h * n;
    const float u = ldf(p + i), v = ldf(p + half + i);
    stf(p + i, u * rcs[i] - v * rcs[half + i]);
    stf(p + half + i, v * rcs[i] + u * rcs[half + i]);
  }
}

int rotate_heads_halves(void* x, int ldx, const int32_t* positions, const double* freq, int T, int H, int n, float sign, int elt, cudaStream_t st) {
  if (T <= 0 || n < 2) return 0;
  KGE_REQUIRE(n % 2 == 0 && freq, "rotate_heads_halves: %d dimensions", n);
  cudaError_t ce = elt == KGE_ELT_F32 ? launch_pdl(rotate_heads_halves_kernel<float>, dim3(T), dim3(256), (size_t)n * 4, st, (float*)x, ldx, positions, freq, H, n, sign)
                                      : launch_pdl(rotate_heads_halves_kernel<__nv_bfloat16>, dim3(T), dim3(256), (size_t)n * 4, st, (__nv_bfloat16*)x, ldx, positions, freq, H, n, sign);
  KGE_CUDA_OK(ce);
  return 0;
}

}  // namespace kge
