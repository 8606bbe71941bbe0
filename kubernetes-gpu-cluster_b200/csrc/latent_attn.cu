// Attention through latents, the row-wise parts around the attention kernel: the RMS norms of the down-projected
// latents, the rotation of the rotated query / key parts with the assembly of every head's key and value rows in the
// paged caches (a head's key is its own up-projected part followed by the one rotated part all heads share), and the
// sigmoid output gate.  One block per token; norms and angles in fp32 / double, one rounding into the storage type.
#include <math.h>

#include "common.cuh"
#include "elt_access.cuh"
#include "hybrid_ops.h"

namespace kge {

__device__ __forceinline__ void sincos_turns(double ang, float* s, float* c) {
  const double turns = rint(ang * 0.15915494309189535);
  sincosf((float)fma(-turns, 6.283185307179586, ang), s, c);
}

template <typename E>
__global__ void __launch_bounds__(256) segment_rmsnorm_kernel(SegNormArgs a) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float red[33];
  const int t = blockIdx.x;
  for (int g = 0; g < a.nseg; ++g) {
    const E* x = (const E*)a.x + (int64_t)t * a.ldx + a.col[g];
    const int n = a.n[g];
    float ss = 0.f;
    for (int c = threadIdx.x; c < n; c += blockDim.x) { const float v = ldf(x + c); ss = fmaf(v, v, ss); }
    const float inv = 1.f / sqrtf(block_sum(ss, red) / (float)n + a.eps);
    E* y = (E*)a.out[g] + (int64_t)t * a.ldo[g];
    for (int c = threadIdx.x; c < n; c += blockDim.x) stf(y + c, ldf(x + c) * inv * ldf((const E*)a.w[g] + c));
  }
}

// the same with one warp per (token, range) and four columns per load: a range of up to 1024 columns stays in the
// warp's registers between the sum of squares and the write, and nothing waits on a barrier
template <typename E>
__global__ void __launch_bounds__(256) segment_rmsnorm_vec_kernel(SegNormArgs a) {
  pdl_launch_dependents();
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const int64_t item = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (item >= (int64_t)a.T * a.nseg) return;
  const int t = (int)(item / a.nseg), g = (int)(item % a.nseg);
  const E* x = (const E*)a.x + (int64_t)t * a.ldx + a.col[g];
  const int n = a.n[g];
  float v[8][4];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int c = (i * 32 + lane) * 4;
    if (c < n) {
      ld4(x + c, v[i]);
      ss = fmaf(v[i][0], v[i][0], fmaf(v[i][1], v[i][1], fmaf(v[i][2], v[i][2], fmaf(v[i][3], v[i][3], ss))));
    }
  }
  const float inv = 1.f / sqrtf(warp_sum(ss) / (float)n + a.eps);
  E* y = (E*)a.out[g] + (int64_t)t * a.ldo[g];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int c = (i * 32 + lane) * 4;
    if (c < n) {
      float w[4];
      ld4((const E*)a.w[g] + c, w);
#pragma unroll
      for (int k = 0; k < 4; ++k) w[k] = v[i][k] * inv * w[k];
      st4(y + c, w);
    }
  }
}

int segment_rmsnorm(const SegNormArgs& a, cudaStream_t st) {
  if (a.T <= 0 || a.nseg <= 0) return 0;
  KGE_REQUIRE(a.nseg <= 2, "segment_rmsnorm: %d segments", a.nseg);
  bool vec = a.ldx % 8 == 0 && (reinterpret_cast<uintptr_t>(a.x) & 15) == 0;
  for (int g = 0; g < a.nseg; ++g)
    vec = vec && a.n[g] <= 1024 && a.n[g] % 8 == 0 && a.col[g] % 8 == 0 && a.ldo[g] % 8 == 0 && ((reinterpret_cast<uintptr_t>(a.w[g]) | reinterpret_cast<uintptr_t>(a.out[g])) & 15) == 0;
  if (vec) {
    const unsigned blocks = (unsigned)(((int64_t)a.T * a.nseg + 7) / 8);
    KGE_CUDA_OK(a.elt == KGE_ELT_F32 ? launch_pdl(segment_rmsnorm_vec_kernel<float>, dim3(blocks), dim3(256), 0, st, a)
                                     : launch_pdl(segment_rmsnorm_vec_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, st, a));
    return 0;
  }
  cudaError_t ce = a.elt == KGE_ELT_F32 ? launch_pdl(segment_rmsnorm_kernel<float>, dim3(a.T), dim3(256), 0, st, a)
                                        : launch_pdl(segment_rmsnorm_kernel<__nv_bfloat16>, dim3(a.T), dim3(256), 0, st, a);
  KGE_CUDA_OK(ce);
  return 0;
}

template <typename E>
__global__ void __launch_bounds__(256) latent_rotary_kvwrite_kernel(LatentKvArgs a) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ float sm[];                 // [half] cos, [half] sin, [rot_part] the turned shared key part
  const int t = blockIdx.x, half = a.rot_dims >> 1, nope = a.dim - a.rot_part;
  float* cs = sm;
  float* kr = sm + 2 * half;
  const int pos = a.positions[t];
  for (int i = threadIdx.x; i < half; i += blockDim.x) {
    float s, c;
    sincos_turns((double)pos * a.freq[i], &s, &c);
    cs[i] = c; cs[half + i] = s;
  }
  __syncthreads();
  // the shared key part: pairs of the first rot_dims turn, the rest passes; rounded once into the storage type
  const E* krs = (const E*)a.k_rot + (int64_t)t * a.ldr;
  for (int i = threadIdx.x; i < a.rot_part; i += blockDim.x) {
    float v;
    if (i < a.rot_dims) {
      const int pr = i >> 1;
      const float u0 = ldf(krs + 2 * pr), u1 = ldf(krs + 2 * pr + 1);
      v = (i & 1) ? fmaf(u1, cs[pr], u0 * cs[half + pr]) : fmaf(u0, cs[pr], -u1 * cs[half + pr]);
    } else v = ldf(krs + i);
    kr[i] = rnd<E>(v);
  }
  // queries in place: one item = one pair of one head
  E* q = (E*)a.q + (int64_t)t * a.ldq;
  for (int it = threadIdx.x; it < a.H * half; it += blockDim.x) {
    const int h = it / half, pr = it % half;
    E* p = q + (int64_t)h * a.dim + nope + 2 * pr;
    const float u0 = ldf(p), u1 = ldf(p + 1);
    stf(p, fmaf(u0, cs[pr], -u1 * cs[half + pr]));
    stf(p + 1, fmaf(u1, cs[pr], u0 * cs[half + pr]));
  }
  __syncthreads();
  const int64_t slot = a.slots ? a.slots[t] : -1;
  if (slot < 0) return;
  const int64_t blk = slot / a.block_size, off = slot % a.block_size;
  E* kc = (E*)a.k_cache;
  E* vc = (E*)a.v_cache;
  const E* kn = (const E*)a.k_nope + (int64_t)t * a.ldk;
  const E* v = (const E*)a.v + (int64_t)t * a.ldv;
  constexpr int VE = 16 / (int)sizeof(E);           // elements per 16-byte piece
  if (a.vec) {
    // 16-byte pieces: a head's own key part and its value straight from the up-projection, the shared part from shared memory
    const int kp = a.dim / VE, vp = a.vdim / VE;
    for (int c = threadIdx.x; c < a.H * kp; c += blockDim.x) {
      const int h = c / kp, d = (c % kp) * VE;
      E* dst = kc + ((blk * a.H + h) * a.block_size + off) * a.dim + d;
      if (d < nope) *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(kn + (int64_t)h * nope + d);
      else {
        __align__(16) E tmp[VE];
#pragma unroll
        for (int i = 0; i < VE; ++i) stf(tmp + i, kr[d - nope + i]);
        *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(tmp);
      }
    }
    for (int c = threadIdx.x; c < a.H * vp; c += blockDim.x) {
      const int h = c / vp, d = (c % vp) * VE;
      *reinterpret_cast<uint4*>(vc + ((blk * a.H + h) * a.block_size + off) * a.vdim + d) = *reinterpret_cast<const uint4*>(v + (int64_t)h * a.vdim + d);
    }
    return;
  }
  for (int c = threadIdx.x; c < a.H * a.dim; c += blockDim.x) {
    const int h = c / a.dim, d = c % a.dim;
    E* dst = kc + ((blk * a.H + h) * a.block_size + off) * a.dim + d;
    if (d < nope) *dst = kn[(int64_t)h * nope + d];
    else stf(dst, kr[d - nope]);
  }
  for (int c = threadIdx.x; c < a.H * a.vdim; c += blockDim.x) {
    const int h = c / a.vdim, d = c % a.vdim;
    vc[((blk * a.H + h) * a.block_size + off) * a.vdim + d] = v[c];
  }
}

int latent_rotary_kvwrite(const LatentKvArgs& a, cudaStream_t st) {
  if (a.T <= 0) return 0;
  KGE_REQUIRE(a.rot_dims % 2 == 0 && a.rot_dims <= a.rot_part && a.rot_part <= a.dim && (a.rot_dims == 0 || a.freq), "latent_rotary_kvwrite: bad rotary sizes");
  const size_t smem = (size_t)(a.rot_dims + a.rot_part) * 4 + 16;
  LatentKvArgs b = a;
  const int ve = a.elt == KGE_ELT_F32 ? 4 : 8;
  b.vec = (a.dim - a.rot_part) % ve == 0 && a.rot_part % ve == 0 && a.vdim % ve == 0 && a.ldk % ve == 0 && a.ldv % ve == 0 &&
          ((reinterpret_cast<uintptr_t>(a.k_nope) | reinterpret_cast<uintptr_t>(a.v) | reinterpret_cast<uintptr_t>(a.k_cache) | reinterpret_cast<uintptr_t>(a.v_cache)) & 15) == 0;
  cudaError_t ce = a.elt == KGE_ELT_F32 ? launch_pdl(latent_rotary_kvwrite_kernel<float>, dim3(a.T), dim3(256), smem, st, b)
                                        : launch_pdl(latent_rotary_kvwrite_kernel<__nv_bfloat16>, dim3(a.T), dim3(256), smem, st, b);
  KGE_CUDA_OK(ce);
  return 0;
}

template <typename E>
__global__ void __launch_bounds__(256) sigmoid_gate_mul_kernel(E* y, int ldy, const E* g, int ldg, int n) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  for (int c = threadIdx.x; c < n; c += blockDim.x) {
    E* p = y + (int64_t)t * ldy + c;
    stf(p, ldf(p) / (1.f + expf(-ldf(g + (int64_t)t * ldg + c))));
  }
}

int sigmoid_gate_mul(void* y, int ldy, const void* g, int ldg, int T, int n, int elt, cudaStream_t st) {
  if (T <= 0) return 0;
  cudaError_t ce = elt == KGE_ELT_F32 ? launch_pdl(sigmoid_gate_mul_kernel<float>, dim3(T), dim3(256), 0, st, (float*)y, ldy, (const float*)g, ldg, n)
                                      : launch_pdl(sigmoid_gate_mul_kernel<__nv_bfloat16>, dim3(T), dim3(256), 0, st, (__nv_bfloat16*)y, ldy, (const __nv_bfloat16*)g, ldg, n);
  KGE_CUDA_OK(ce);
  return 0;
}

}  // namespace kge
