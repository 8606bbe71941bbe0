// WKV token mixing for layer-list models: every projection reads its own blend of a token's row and the row before it
// ("token shift"), and each head carries a dim x dim matrix S in fp32 that decays per key channel and per token:
//     o_t = (S + diag(u) k_t v_t^T)^T r_t,      S <- diag(w_t) S + k_t v_t^T,      w_t = exp(-exp(decay_pre_t))
// The previous row and S live in the request's state slot, so a prompt cut anywhere continues exactly: the recurrence
// walks a request's rows in order, one thread per value column with its column of S in registers.
#include <algorithm>

#include "common.cuh"
#include "elt_access.cuh"
#include "hybrid_ops.h"

namespace kge {

// One block per token.  The row before a request's first row of this step comes from the slot (zeros at position 0);
// nothing is written to the slot here, so the blocks of a request do not race with it.
template <typename E>
__global__ void __launch_bounds__(256) wkv_shift_mix_kernel(WkvArgs a) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x, b = a.token_req[t], d = a.d;
  const bool first = t == a.qsl[b];
  const bool zero = first && a.positions[t] == 0;
  const E* h = (const E*)a.h + (int64_t)t * a.ldh;
  const E* hp = (const E*)a.h + (int64_t)(t - 1) * a.ldh;
  const float* sp = a.state + (int64_t)a.slots[b] * a.slot_stride;
  for (int c = threadIdx.x; c < d; c += blockDim.x) {
    const float x = ldf(h + c);
    const float p = zero ? 0.f : (first ? sp[c] : ldf(hp + c));
    const float dx = p - x;
    for (int z = 0; z < a.nmix; ++z) stf((E*)a.mixes + ((int64_t)z * a.T + t) * d + c, fmaf(dx, ldf((const E*)a.mu + (int64_t)z * d + c), x));
  }
}

// after the blends: the slot keeps the last row of every request of the step
template <typename E>
__global__ void __launch_bounds__(256) wkv_save_row_kernel(WkvArgs a) {
  pdl_launch_dependents();
  pdl_wait();
  const int b = blockIdx.x, last = a.qsl[b + 1] - 1;
  if (last < a.qsl[b]) return;
  const E* h = (const E*)a.h + (int64_t)last * a.ldh;
  float* sp = a.state + (int64_t)a.slots[b] * a.slot_stride;
  for (int c = threadIdx.x; c < a.d; c += blockDim.x) sp[c] = ldf(h + c);
}

int wkv_shift_mix(const WkvArgs& a, cudaStream_t st) {
  if (a.T <= 0) return 0;
  if (a.elt == KGE_ELT_F32) {
    KGE_CUDA_OK(launch_pdl(wkv_shift_mix_kernel<float>, dim3(a.T), dim3(256), 0, st, a));
    KGE_CUDA_OK(launch_pdl(wkv_save_row_kernel<float>, dim3(a.B), dim3(256), 0, st, a));
  } else {
    KGE_CUDA_OK(launch_pdl(wkv_shift_mix_kernel<__nv_bfloat16>, dim3(a.T), dim3(256), 0, st, a));
    KGE_CUDA_OK(launch_pdl(wkv_save_row_kernel<__nv_bfloat16>, dim3(a.B), dim3(256), 0, st, a));
  }
  return 0;
}

// One block per (request, head): thread j owns value column j and the column S[:, j] in registers; the token's r, k and
// decay (dim numbers each) pass through a double-buffered shared tile, one barrier per token, the next token's operands
// being requested while the current one is computed.
template <typename E, int MAXD>
__global__ void __launch_bounds__(MAXD) wkv_scan_kernel(WkvArgs a) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ __align__(16) float rs[2][MAXD], ks[2][MAXD], ws[2][MAXD], us[MAXD];
  const int b = blockIdx.x, h = blockIdx.y, j = threadIdx.x, dim = a.dim, HD = a.H * a.dim;
  const int r0 = a.qsl[b], r1 = a.qsl[b + 1];
  if (r0 >= r1) return;
  const bool on = j < dim;
  const bool fresh = a.positions[r0] == 0;
  float* Sg = a.state + (int64_t)a.slots[b] * a.slot_stride + a.d + (int64_t)h * dim * dim;
  float S[MAXD];
#pragma unroll
  for (int i = 0; i < MAXD; ++i) S[i] = (i < dim && on && !fresh) ? Sg[(int64_t)i * dim + j] : 0.f;
  us[j] = on ? a.u[h * dim + j] : 0.f;
  const E *rp = (const E*)a.r, *kp = (const E*)a.k, *vp = (const E*)a.v;
  float rn = 0.f, kn = 0.f, wn = 0.f, vn = 0.f;
  auto fetch = [&](int t) {
    if (on) {
      const int64_t o = (int64_t)t * a.ld + h * dim + j;
      rn = ldf(rp + o); kn = ldf(kp + o); vn = ldf(vp + o);
      wn = a.decay_pre[(int64_t)t * HD + h * dim + j];
    }
  };
  fetch(r0);
  for (int t = r0; t < r1; ++t) {
    const int p = (t - r0) & 1;
    rs[p][j] = rn; ks[p][j] = kn; ws[p][j] = expf(-expf(wn));
    const float v = vn;
    if (t + 1 < r1) fetch(t + 1);
    __syncthreads();
    float acc0 = 0.f, acc1 = 0.f, acc2 = 0.f, acc3 = 0.f;
#pragma unroll
    for (int i4 = 0; i4 < MAXD / 4; ++i4) {
      if (i4 * 4 < dim) {
        const float4 r4 = reinterpret_cast<const float4*>(rs[p])[i4], k4 = reinterpret_cast<const float4*>(ks[p])[i4];
        const float4 w4 = reinterpret_cast<const float4*>(ws[p])[i4], u4 = reinterpret_cast<const float4*>(us)[i4];
        float kv;
        kv = k4.x * v; acc0 = fmaf(r4.x, fmaf(u4.x, kv, S[i4 * 4 + 0]), acc0); S[i4 * 4 + 0] = fmaf(w4.x, S[i4 * 4 + 0], kv);
        kv = k4.y * v; acc1 = fmaf(r4.y, fmaf(u4.y, kv, S[i4 * 4 + 1]), acc1); S[i4 * 4 + 1] = fmaf(w4.y, S[i4 * 4 + 1], kv);
        kv = k4.z * v; acc2 = fmaf(r4.z, fmaf(u4.z, kv, S[i4 * 4 + 2]), acc2); S[i4 * 4 + 2] = fmaf(w4.z, S[i4 * 4 + 2], kv);
        kv = k4.w * v; acc3 = fmaf(r4.w, fmaf(u4.w, kv, S[i4 * 4 + 3]), acc3); S[i4 * 4 + 3] = fmaf(w4.w, S[i4 * 4 + 3], kv);
      }
    }
    if (on) a.o32[(int64_t)t * HD + h * dim + j] = (acc0 + acc1) + (acc2 + acc3);
  }
  if (on) {
#pragma unroll
    for (int i = 0; i < MAXD; ++i) if (i < dim) Sg[(int64_t)i * dim + j] = S[i];
  }
}

// one warp per (token, head): o / rms(o) * norm_w * silu(gate_pre)
template <typename E>
__global__ void __launch_bounds__(256) wkv_norm_gate_kernel(WkvArgs a) {
  pdl_launch_dependents();
  pdl_wait();
  const int64_t item = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (item >= (int64_t)a.T * a.H) return;
  const int lane = threadIdx.x & 31, t = (int)(item / a.H), h = (int)(item % a.H), dim = a.dim, HD = a.H * a.dim;
  const float* o = a.o32 + (int64_t)t * HD + h * dim;
  float ss = 0.f;
  for (int c = lane; c < dim; c += 32) ss = fmaf(o[c], o[c], ss);
  const float inv = 1.f / sqrtf(warp_sum(ss) / (float)dim + a.eps);
  const E* g = (const E*)a.gate_pre + (int64_t)t * a.ld + h * dim;
  E* y = (E*)a.out + (int64_t)t * a.ldo + h * dim;
  for (int c = lane; c < dim; c += 32) {
    const float gv = ldf(g + c);
    stf(y + c, o[c] * inv * ldf((const E*)a.norm_w + h * dim + c) * (gv / (1.f + expf(-gv))));
  }
}

template <typename E>
static int wkv_scan_t(const WkvArgs& a, cudaStream_t st) {
  const dim3 grid(a.B, a.H);
  cudaError_t ce;
  if (a.dim <= 32) ce = launch_pdl(wkv_scan_kernel<E, 32>, grid, dim3(32), 0, st, a);
  else if (a.dim <= 64) ce = launch_pdl(wkv_scan_kernel<E, 64>, grid, dim3(64), 0, st, a);
  else if (a.dim <= 128) ce = launch_pdl(wkv_scan_kernel<E, 128>, grid, dim3(128), 0, st, a);
  else ce = launch_pdl(wkv_scan_kernel<E, 256>, grid, dim3(256), 0, st, a);
  KGE_CUDA_OK(ce);
  const int64_t items = (int64_t)a.T * a.H;
  KGE_CUDA_OK(launch_pdl(wkv_norm_gate_kernel<E>, dim3((unsigned)((items + 7) / 8)), dim3(256), 0, st, a));
  return 0;
}

int wkv_scan(const WkvArgs& a, cudaStream_t st) {
  if (a.T <= 0) return 0;
  KGE_REQUIRE(a.dim > 0 && a.dim <= 256 && a.B <= 65535 * 32 && a.H <= 65535, "wkv_scan: head size %d (1 .. 256)", a.dim);
  return a.elt == KGE_ELT_F32 ? wkv_scan_t<float>(a, st) : wkv_scan_t<__nv_bfloat16>(a, st);
}

}  // namespace kge
