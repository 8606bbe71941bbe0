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

// the decay of a key channel from its logit: exp(-exp(z)), or (mode 1) sigmoid(z)^(1 / tau); log_decay is its natural logarithm
__device__ __forceinline__ float log_decay(float z, int mode, float tau) {
  if (mode == 0) return -expf(z);
  const float ls = z < 0.f ? z - log1pf(expf(z)) : -log1pf(expf(-z));      // log(sigmoid(z)) without overflow on either side
  return ls / tau;
}

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

// the same, four columns per thread and pass (rows of 16-byte multiples)
template <typename E>
__global__ void __launch_bounds__(256) wkv_shift_mix_vec_kernel(WkvArgs a) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x, b = a.token_req[t], d = a.d;
  const bool first = t == a.qsl[b];
  const bool zero = first && a.positions[t] == 0;
  const E* h = (const E*)a.h + (int64_t)t * a.ldh;
  const E* hp = (const E*)a.h + (int64_t)(t - 1) * a.ldh;
  const float* sp = a.state + (int64_t)a.slots[b] * a.slot_stride;
  for (int c = threadIdx.x * 4; c < d; c += blockDim.x * 4) {
    float x[4], p[4] = {0.f, 0.f, 0.f, 0.f}, m[4], o[4];
    ld4(h + c, x);
    if (!zero) { if (first) ld4(sp + c, p); else ld4(hp + c, p); }
    for (int z = 0; z < a.nmix; ++z) {
      ld4((const E*)a.mu + (int64_t)z * d + c, m);
#pragma unroll
      for (int i = 0; i < 4; ++i) o[i] = fmaf(p[i] - x[i], m[i], x[i]);
      st4((E*)a.mixes + ((int64_t)z * a.T + t) * d + c, o);
    }
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
  const bool vec = a.d % 8 == 0 && a.ldh % 8 == 0 && a.slot_stride % 4 == 0 && ((reinterpret_cast<uintptr_t>(a.h) | reinterpret_cast<uintptr_t>(a.mu) | reinterpret_cast<uintptr_t>(a.mixes) | reinterpret_cast<uintptr_t>(a.state)) & 15) == 0;
  if (vec) {
    cudaError_t ce = a.elt == KGE_ELT_F32 ? launch_pdl(wkv_shift_mix_vec_kernel<float>, dim3(a.T), dim3(256), 0, st, a)
                                          : launch_pdl(wkv_shift_mix_vec_kernel<__nv_bfloat16>, dim3(a.T), dim3(256), 0, st, a);
    KGE_CUDA_OK(ce);
    ce = a.elt == KGE_ELT_F32 ? launch_pdl(wkv_save_row_kernel<float>, dim3(a.B), dim3(256), 0, st, a) : launch_pdl(wkv_save_row_kernel<__nv_bfloat16>, dim3(a.B), dim3(256), 0, st, a);
    KGE_CUDA_OK(ce);
    return 0;
  }
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
  const int b = blockIdx.x, h = blockIdx.y, j = threadIdx.x, dim = a.dim, vd = a.vdim > 0 ? a.vdim : a.dim, HD = a.H * a.dim, HDv = a.H * vd;
  const int r0 = a.qsl[b], r1 = a.qsl[b + 1];
  if (r0 >= r1) return;
  const bool onk = j < dim, on = j < vd;            // this thread's key channel (operands) and value column (state, output)
  const bool fresh = a.positions[r0] == 0;
  const bool after = a.read_after;
  float* Sg = a.state + (int64_t)a.slots[b] * a.slot_stride + a.d + (int64_t)h * dim * vd;
  float S[MAXD];
#pragma unroll
  for (int i = 0; i < MAXD; ++i) S[i] = (i < dim && on && !fresh) ? Sg[(int64_t)i * vd + j] : 0.f;
  us[j] = (onk && a.u) ? a.u[h * dim + j] : 0.f;
  const E *rp = (const E*)a.r, *kp = (const E*)a.k, *vp = (const E*)a.v;
  float rn = 0.f, kn = 0.f, wn = 0.f, vn = 0.f;
  auto fetch = [&](int t) {
    if (onk) {
      const int64_t o = (int64_t)t * a.ld + h * dim + j;
      rn = ldf(rp + o) * a.r_scale; kn = ldf(kp + o);
      wn = a.decay_pre[(int64_t)t * HD + h * dim + j];
    }
    if (on) vn = ldf(vp + (int64_t)t * a.ld + h * vd + j);
  };
  fetch(r0);
  for (int t = r0; t < r1; ++t) {
    const int p = (t - r0) & 1;
    rs[p][j] = rn; ks[p][j] = kn; ws[p][j] = expf(log_decay(wn, a.decay_mode, a.tau));
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
        if (after) {                                 // the read-out sees the state after this token's update
          S[i4 * 4 + 0] = fmaf(w4.x, S[i4 * 4 + 0], k4.x * v); acc0 = fmaf(r4.x, S[i4 * 4 + 0], acc0);
          S[i4 * 4 + 1] = fmaf(w4.y, S[i4 * 4 + 1], k4.y * v); acc1 = fmaf(r4.y, S[i4 * 4 + 1], acc1);
          S[i4 * 4 + 2] = fmaf(w4.z, S[i4 * 4 + 2], k4.z * v); acc2 = fmaf(r4.z, S[i4 * 4 + 2], acc2);
          S[i4 * 4 + 3] = fmaf(w4.w, S[i4 * 4 + 3], k4.w * v); acc3 = fmaf(r4.w, S[i4 * 4 + 3], acc3);
        } else {
        kv = k4.x * v; acc0 = fmaf(r4.x, fmaf(u4.x, kv, S[i4 * 4 + 0]), acc0); S[i4 * 4 + 0] = fmaf(w4.x, S[i4 * 4 + 0], kv);
        kv = k4.y * v; acc1 = fmaf(r4.y, fmaf(u4.y, kv, S[i4 * 4 + 1]), acc1); S[i4 * 4 + 1] = fmaf(w4.y, S[i4 * 4 + 1], kv);
        kv = k4.z * v; acc2 = fmaf(r4.z, fmaf(u4.z, kv, S[i4 * 4 + 2]), acc2); S[i4 * 4 + 2] = fmaf(w4.z, S[i4 * 4 + 2], kv);
        kv = k4.w * v; acc3 = fmaf(r4.w, fmaf(u4.w, kv, S[i4 * 4 + 3]), acc3); S[i4 * 4 + 3] = fmaf(w4.w, S[i4 * 4 + 3], kv);
        }
      }
    }
    if (on) a.o32[(int64_t)t * HDv + h * vd + j] = (acc0 + acc1) + (acc2 + acc3);
  }
  if (on) {
#pragma unroll
    for (int i = 0; i < MAXD; ++i) if (i < dim) Sg[(int64_t)i * vd + j] = S[i];
  }
}

// Prompt steps: the same recurrence 32 tokens at a time, in fp32 on the CUDA cores.  With L_t the running sum of the log
// decays inside the chunk (L_-1 = 0) and S the state at the chunk's start,
//     o_t = sum_k r_tk e^{L_(t-1)k} S_k. + sum_{j<t} (sum_k r_tk k_jk e^{L_(t-1)k - L_jk}) v_j + (sum_k r_tk u_k k_tk) v_t
//     S  <- diag(e^{L_last}) S + sum_j (k_j e^{L_last - L_j}) v_j^T
// Every exponent is a sum of log decays of tokens between the two positions, so it is <= 0 and nothing overflows however
// fast a channel forgets.  One block of 256 threads per (request, head), head sizes up to 64 (a multiple of 4): the
// read-out and the state update are 2 x 4 / 4 x 4 register tiles over shared operands; the state stays in registers
// across chunks (mirrored in shared memory for the read-out).  A request's last chunk may be short.
constexpr int WC = 32, WD = 64, WLD = WD + 4, WLC = WC + 4;
constexpr size_t WKV_CHUNK_SMEM = (size_t)(5 * WC * WLD + WD * WLC + WC * WLC + WD * WLD + 2 * WD) * 4;

template <typename E>
__global__ void __launch_bounds__(256) wkv_chunk_kernel(WkvArgs a) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ __align__(16) float sm[];
  float* rs = sm;                       // [WC][WLD] r
  float* ks = rs + WC * WLD;            // [WC][WLD] k
  float* vs = ks + WC * WLD;            // [WC][WLD] v
  float* Ls = vs + WC * WLD;            // [WC][WLD] log decays (in units of log 2), then their running sums
  float* kd = Ls + WC * WLD;            // [WC][WLD] k_j e^{L_last - L_j}
  float* rdT = kd + WC * WLD;           // [WD][WLC] r_t e^{L_(t-1)}, transposed
  float* PT = rdT + WD * WLC;           // [WC][WLC] scores, transposed: PT[j][t]
  float* Ss = PT + WC * WLC;            // [WD][WLD] the state at the chunk's start
  float* us = Ss + WD * WLD;            // [WD] bonus
  float* el = us + WD;                  // [WD] e^{L_last}
  const int b = blockIdx.x, h = blockIdx.y, tid = threadIdx.x, dim = a.dim, vd = a.vdim > 0 ? a.vdim : a.dim, HD = a.H * a.dim, HDv = a.H * vd;
  const int r0 = a.qsl[b], r1 = a.qsl[b + 1];
  if (r0 >= r1) return;
  const bool fresh = a.positions[r0] == 0;
  const int inc = a.read_after ? 1 : 0;            // 1: token t reads the state after its own update (L_t in place of L_(t-1), no bonus)
  float* Sg = a.state + (int64_t)a.slots[b] * a.slot_stride + a.d + (int64_t)h * dim * vd;
  const int kg = tid >> 4, vg = tid & 15;          // this thread's state tile: rows kg * 4 .., columns vg * 4 ..
  float S[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int k = kg * 4 + i, v = vg * 4 + j;
      S[i][j] = (!fresh && k < dim && v < vd) ? Sg[(int64_t)k * vd + v] : 0.f;
    }
  if (tid < WD) us[tid] = (tid < dim && a.u) ? a.u[h * dim + tid] : 0.f;
  const E *rp = (const E*)a.r, *kp = (const E*)a.k, *vp = (const E*)a.v;
  for (int c0 = r0; c0 < r1; c0 += WC) {
    const int n = min(WC, r1 - c0);
    __syncthreads();                               // the previous chunk's readers are done
    for (int i = tid; i < WC * WD; i += 256) {
      const int t = i / WD, c = i % WD;
      const bool ok = t < n && c < dim;
      const int64_t o = (int64_t)(c0 + t) * a.ld + h * dim + c;
      rs[t * WLD + c] = ok ? ldf(rp + o) * a.r_scale : 0.f;
      ks[t * WLD + c] = ok ? ldf(kp + o) : 0.f;
      vs[t * WLD + c] = (t < n && c < vd) ? ldf(vp + (int64_t)(c0 + t) * a.ld + h * vd + c) : 0.f;
      Ls[t * WLD + c] = ok ? log_decay(a.decay_pre[(int64_t)(c0 + t) * HD + h * dim + c], a.decay_mode, a.tau) * 1.4426950408889634f : 0.f;
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) *reinterpret_cast<float4*>(Ss + (kg * 4 + i) * WLD + vg * 4) = make_float4(S[i][0], S[i][1], S[i][2], S[i][3]);
    __syncthreads();
    if (tid < WD) {                                // running sums per channel
      float acc = 0.f;
#pragma unroll 8
      for (int t = 0; t < WC; ++t) { acc += Ls[t * WLD + tid]; Ls[t * WLD + tid] = acc; }
      el[tid] = exp2f(acc);
    }
    __syncthreads();
    for (int i = tid; i < WC * WD; i += 256) {
      const int t = i / WD, c = i % WD;
      const float lm1 = t + inc > 0 ? Ls[(t - 1 + inc) * WLD + c] : 0.f;
      rdT[c * WLC + t] = rs[t * WLD + c] * exp2f(lm1);
      kd[t * WLD + c] = ks[t * WLD + c] * exp2f(Ls[(WC - 1) * WLD + c] - Ls[t * WLD + c]);
    }
    {
      // scores: thread (t, j mod 8) walks its keys j <= t
      const int t = tid >> 3, jq = tid & 7;
      const float* rt = rs + t * WLD;
      const float* lt = Ls + (t - 1 + inc) * WLD;  // read only for j < t + inc, so the row exists
      for (int j = jq; j < WC; j += 8) {
        float acc = 0.f;
        if (j < t + inc) {
          const float *kj = ks + j * WLD, *lj = Ls + j * WLD;
#pragma unroll 4
          for (int c = 0; c < WD; c += 4) {
            const float4 r4 = *reinterpret_cast<const float4*>(rt + c), k4 = *reinterpret_cast<const float4*>(kj + c);
            const float4 a4 = *reinterpret_cast<const float4*>(lt + c), b4 = *reinterpret_cast<const float4*>(lj + c);
            acc = fmaf(r4.x * k4.x, exp2f(a4.x - b4.x), acc); acc = fmaf(r4.y * k4.y, exp2f(a4.y - b4.y), acc);
            acc = fmaf(r4.z * k4.z, exp2f(a4.z - b4.z), acc); acc = fmaf(r4.w * k4.w, exp2f(a4.w - b4.w), acc);
          }
        } else if (j == t) {
          const float* kj = ks + j * WLD;
#pragma unroll 4
          for (int c = 0; c < WD; c += 4) {
            const float4 r4 = *reinterpret_cast<const float4*>(rt + c), k4 = *reinterpret_cast<const float4*>(kj + c), u4 = *reinterpret_cast<const float4*>(us + c);
            acc = fmaf(r4.x * u4.x, k4.x, acc); acc = fmaf(r4.y * u4.y, k4.y, acc); acc = fmaf(r4.z * u4.z, k4.z, acc); acc = fmaf(r4.w * u4.w, k4.w, acc);
          }
        }
        PT[j * WLC + t] = acc;
      }
    }
    __syncthreads();
    {
      // read-out: rows tg * 2 .., columns vg * 4 ..: the carried state, then the chunk's own keys
      const int tg = tid >> 4;
      float o[2][4] = {};
#pragma unroll 8
      for (int k = 0; k < WD; ++k) {
        const float2 r2 = *reinterpret_cast<const float2*>(rdT + k * WLC + tg * 2);
        const float4 s4 = *reinterpret_cast<const float4*>(Ss + k * WLD + vg * 4);
        o[0][0] = fmaf(r2.x, s4.x, o[0][0]); o[0][1] = fmaf(r2.x, s4.y, o[0][1]); o[0][2] = fmaf(r2.x, s4.z, o[0][2]); o[0][3] = fmaf(r2.x, s4.w, o[0][3]);
        o[1][0] = fmaf(r2.y, s4.x, o[1][0]); o[1][1] = fmaf(r2.y, s4.y, o[1][1]); o[1][2] = fmaf(r2.y, s4.z, o[1][2]); o[1][3] = fmaf(r2.y, s4.w, o[1][3]);
      }
      const int jmax = min(tg * 2 + 2, n);
      for (int j = 0; j < jmax; ++j) {
        const float2 p2 = *reinterpret_cast<const float2*>(PT + j * WLC + tg * 2);
        const float4 v4 = *reinterpret_cast<const float4*>(vs + j * WLD + vg * 4);
        o[0][0] = fmaf(p2.x, v4.x, o[0][0]); o[0][1] = fmaf(p2.x, v4.y, o[0][1]); o[0][2] = fmaf(p2.x, v4.z, o[0][2]); o[0][3] = fmaf(p2.x, v4.w, o[0][3]);
        o[1][0] = fmaf(p2.y, v4.x, o[1][0]); o[1][1] = fmaf(p2.y, v4.y, o[1][1]); o[1][2] = fmaf(p2.y, v4.z, o[1][2]); o[1][3] = fmaf(p2.y, v4.w, o[1][3]);
      }
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        const int t = tg * 2 + i;
        if (t < n && vg * 4 < vd) *reinterpret_cast<float4*>(a.o32 + (int64_t)(c0 + t) * HDv + h * vd + vg * 4) = make_float4(o[i][0], o[i][1], o[i][2], o[i][3]);
      }
    }
    {
      // the state moves to the chunk's end
      const float4 e4 = *reinterpret_cast<const float4*>(el + kg * 4);
      const float ee[4] = {e4.x, e4.y, e4.z, e4.w};
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) S[i][j] *= ee[i];
#pragma unroll 4
      for (int j = 0; j < n; ++j) {
        const float4 k4 = *reinterpret_cast<const float4*>(kd + j * WLD + kg * 4);
        const float4 v4 = *reinterpret_cast<const float4*>(vs + j * WLD + vg * 4);
        const float kk[4] = {k4.x, k4.y, k4.z, k4.w}, vv[4] = {v4.x, v4.y, v4.z, v4.w};
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
          for (int jj = 0; jj < 4; ++jj) S[i][jj] = fmaf(kk[i], vv[jj], S[i][jj]);
      }
    }
  }
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int k = kg * 4 + i, v = vg * 4 + j;
      if (k < dim && v < vd) Sg[(int64_t)k * vd + v] = S[i][j];
    }
}

// one warp per (token, head): o / rms(o) * norm_w * silu(gate_pre)
template <typename E>
__global__ void __launch_bounds__(256) wkv_norm_gate_kernel(WkvArgs a) {
  pdl_launch_dependents();
  pdl_wait();
  const int64_t item = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (item >= (int64_t)a.T * a.H) return;
  const int lane = threadIdx.x & 31, t = (int)(item / a.H), h = (int)(item % a.H), dim = a.vdim > 0 ? a.vdim : a.dim, HD = a.H * dim;
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

// the same with four columns per lane and pass (head sizes and row strides of 4-column multiples, 16-byte aligned rows)
template <typename E>
__global__ void __launch_bounds__(256) wkv_norm_gate_vec_kernel(WkvArgs a) {
  pdl_launch_dependents();
  pdl_wait();
  const int64_t item = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (item >= (int64_t)a.T * a.H) return;
  const int lane = threadIdx.x & 31, t = (int)(item / a.H), h = (int)(item % a.H), dim = a.vdim > 0 ? a.vdim : a.dim, HD = a.H * dim;
  const float* o = a.o32 + (int64_t)t * HD + h * dim;
  float ss = 0.f;
  for (int c = lane * 4; c < dim; c += 128) {
    float v[4];
    ld4(o + c, v);
    ss = fmaf(v[0], v[0], ss); ss = fmaf(v[1], v[1], ss); ss = fmaf(v[2], v[2], ss); ss = fmaf(v[3], v[3], ss);
  }
  const float inv = 1.f / sqrtf(warp_sum(ss) / (float)dim + a.eps);
  const E* g = (const E*)a.gate_pre + (int64_t)t * a.ld + h * dim;
  E* y = (E*)a.out + (int64_t)t * a.ldo + h * dim;
  for (int c = lane * 4; c < dim; c += 128) {
    float v[4], gv[4], w[4], r[4];
    ld4(o + c, v); ld4(g + c, gv); ld4((const E*)a.norm_w + h * dim + c, w);
#pragma unroll
    for (int k = 0; k < 4; ++k) r[k] = v[k] * inv * w[k] * (gv[k] / (1.f + expf(-gv[k])));
    st4(y + c, r);
  }
}

template <typename E>
static int wkv_scan_t(const WkvArgs& a, cudaStream_t st) {
  const dim3 grid(a.B, a.H);
  cudaError_t ce;
  // requests with many rows: 32 tokens at a time (the o32 rows are 16-byte aligned when the head size is a multiple of 4)
  const int vd = a.vdim > 0 ? a.vdim : a.dim, md = std::max(a.dim, vd);
  if (a.max_q >= 8 && a.dim <= WD && a.dim % 4 == 0 && vd <= WD && vd % 4 == 0 && a.H * vd % 4 == 0) {
    static bool smem_set = false;
    if (!smem_set) {
      KGE_CUDA_OK(cudaFuncSetAttribute(wkv_chunk_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)WKV_CHUNK_SMEM));
      KGE_CUDA_OK(cudaFuncSetAttribute(wkv_chunk_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)WKV_CHUNK_SMEM));
      smem_set = true;
    }
    ce = launch_pdl(wkv_chunk_kernel<E>, grid, dim3(256), WKV_CHUNK_SMEM, st, a);
  } else if (md <= 32) ce = launch_pdl(wkv_scan_kernel<E, 32>, grid, dim3(32), 0, st, a);
  else if (md <= 64) ce = launch_pdl(wkv_scan_kernel<E, 64>, grid, dim3(64), 0, st, a);
  else if (md <= 128) ce = launch_pdl(wkv_scan_kernel<E, 128>, grid, dim3(128), 0, st, a);
  else ce = launch_pdl(wkv_scan_kernel<E, 256>, grid, dim3(256), 0, st, a);
  KGE_CUDA_OK(ce);
  const int64_t items = (int64_t)a.T * a.H;
  const bool vec = vd % 4 == 0 && a.ld % 4 == 0 && a.ldo % 4 == 0 &&
                   ((reinterpret_cast<uintptr_t>(a.o32) | reinterpret_cast<uintptr_t>(a.gate_pre) | reinterpret_cast<uintptr_t>(a.out) | reinterpret_cast<uintptr_t>(a.norm_w)) & 15) == 0;
  if (vec) KGE_CUDA_OK(launch_pdl(wkv_norm_gate_vec_kernel<E>, dim3((unsigned)((items + 7) / 8)), dim3(256), 0, st, a));
  else KGE_CUDA_OK(launch_pdl(wkv_norm_gate_kernel<E>, dim3((unsigned)((items + 7) / 8)), dim3(256), 0, st, a));
  return 0;
}

int wkv_scan(const WkvArgs& a, cudaStream_t st) {
  if (a.T <= 0) return 0;
  KGE_REQUIRE(a.dim > 0 && a.dim <= 256 && a.vdim >= 0 && a.vdim <= 256 && a.B <= 65535 * 32 && a.H <= 65535, "wkv_scan: head size %d x %d (1 .. 256)", a.dim, a.vdim);
  KGE_REQUIRE(a.u || a.read_after, "wkv_scan: the read-out before the update needs the bonus vector");
  return a.elt == KGE_ELT_F32 ? wkv_scan_t<float>(a, st) : wkv_scan_t<__nv_bfloat16>(a, st);
}

}  // namespace kge
