// A short causal convolution over time on every channel of a projection, continued across steps from a state slot that
// holds the request's last taps - 1 input rows.  Each output is a sum over the taps in ascending order in fp32, from
// this step's rows or the slot's, so the result does not depend on where a prompt was cut.
#include <algorithm>

#include "common.cuh"
#include "elt_access.cuh"
#include "hybrid_ops.h"

namespace kge {

namespace {

constexpr int SC_MAX_TAPS = 16;

// a block per token and slice of the channels (few tokens: one channel per thread; many: a thread walks its channels);
// a channel's taps are summed in ascending order
template <typename E>
__global__ void __launch_bounds__(256) short_conv_kernel(ShortConvArgs a) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const int b = a.token_req[t], r0 = a.qsl[b], pos = a.positions[t], taps = a.taps;
  const float* sp = a.state + (int64_t)a.slots[b] * a.slot_stride;      // [taps - 1, C]: row s holds the input of position p0 - (taps - 1) + s
  const E* x = (const E*)a.x;
  for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < a.C; c += gridDim.y * blockDim.x) {
    float acc = 0.f;
    for (int j = 0; j < taps; ++j) {
      const int back = taps - 1 - j;                  // the input of position pos - back
      if (pos - back < 0) continue;
      const int row = t - back;
      const float u = row >= r0 ? ldf(x + (int64_t)row * a.ldx + c) : sp[(int64_t)(taps - 1 - (r0 - row)) * a.C + c];
      acc = fmaf(ldf((const E*)a.w + (int64_t)c * taps + j), u, acc);
    }
    stf((E*)a.y + (int64_t)t * a.ldy + c, acc);
  }
}

// the same, four neighbouring channels per thread (8-byte loads of 16-bit rows, 16-byte ones of fp32 rows and of the slot)
template <typename E>
__global__ void __launch_bounds__(256) short_conv_vec_kernel(ShortConvArgs a) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const int b = a.token_req[t], r0 = a.qsl[b], pos = a.positions[t], taps = a.taps;
  const float* sp = a.state + (int64_t)a.slots[b] * a.slot_stride;
  const E* x = (const E*)a.x;
  for (int c = (blockIdx.y * blockDim.x + threadIdx.x) * 4; c < a.C; c += gridDim.y * blockDim.x * 4) {
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    for (int j = 0; j < taps; ++j) {
      const int back = taps - 1 - j;
      if (pos - back < 0) continue;
      const int row = t - back;
      float u[4];
      if (row >= r0) ld4(x + (int64_t)row * a.ldx + c, u); else ld4(sp + (int64_t)(taps - 1 - (r0 - row)) * a.C + c, u);
#pragma unroll
      for (int k = 0; k < 4; ++k) acc[k] = fmaf(ldf((const E*)a.w + (int64_t)(c + k) * taps + j), u[k], acc[k]);
    }
    st4((E*)a.y + (int64_t)t * a.ldy + c, acc);
  }
}

// one block per request: the slot's rows move up by the step's row count and the step's last rows follow
template <typename E>
__global__ void __launch_bounds__(256) short_conv_save_kernel(ShortConvArgs a) {
  pdl_launch_dependents();
  pdl_wait();
  const int b = blockIdx.x, c = blockIdx.y * blockDim.x + threadIdx.x, r0 = a.qsl[b], n = a.qsl[b + 1] - r0, keep = a.taps - 1;
  if (n <= 0 || keep <= 0 || c >= a.C) return;
  const bool fresh = a.positions[r0] == 0;
  float* sp = a.state + (int64_t)a.slots[b] * a.slot_stride;
  const E* x = (const E*)a.x;
  float v[SC_MAX_TAPS];
#pragma unroll
  for (int s = 0; s < SC_MAX_TAPS - 1; ++s) {         // every row is read before any is written
    const int src = s + n;                            // in the old numbering of the slot's rows
    v[s] = 0.f;
    if (s < keep) {
      if (src >= keep) v[s] = ldf(x + (int64_t)(r0 + src - keep) * a.ldx + c);
      else if (!fresh) v[s] = sp[(int64_t)src * a.C + c];
    }
  }
#pragma unroll
  for (int s = 0; s < SC_MAX_TAPS - 1; ++s) if (s < keep) sp[(int64_t)s * a.C + c] = v[s];
}

}  // namespace

int short_conv_state(const ShortConvArgs& a, cudaStream_t st) {
  if (a.T <= 0) return 0;
  KGE_REQUIRE(a.taps >= 1 && a.taps <= SC_MAX_TAPS && a.C > 0 && a.x != a.y, "short_conv_state: %d taps on %d channels", a.taps, a.C);
  const int cb = (a.C + 255) / 256;
  KGE_REQUIRE(cb <= 65535, "short_conv_state: %d channels", a.C);
  const int cy = std::max(1, std::min(cb, 2048 / std::max(a.T, 1)));     // about 2048 blocks at least, else a block per token
  const bool vec = a.C % 4 == 0 && a.ldx % 4 == 0 && a.ldy % 4 == 0 && a.slot_stride % 4 == 0 &&
                   ((reinterpret_cast<uintptr_t>(a.x) | reinterpret_cast<uintptr_t>(a.y) | reinterpret_cast<uintptr_t>(a.state)) & 15) == 0;
  if (vec) {
    const int cv = std::max(1, std::min((a.C / 4 + 255) / 256, 2048 / std::max(a.T, 1)));
    if (a.elt == KGE_ELT_F32) KGE_CUDA_OK(launch_pdl(short_conv_vec_kernel<float>, dim3(a.T, cv), dim3(256), 0, st, a));
    else KGE_CUDA_OK(launch_pdl(short_conv_vec_kernel<__nv_bfloat16>, dim3(a.T, cv), dim3(256), 0, st, a));
    if (a.elt == KGE_ELT_F32) KGE_CUDA_OK(launch_pdl(short_conv_save_kernel<float>, dim3(a.B, cb), dim3(256), 0, st, a));
    else KGE_CUDA_OK(launch_pdl(short_conv_save_kernel<__nv_bfloat16>, dim3(a.B, cb), dim3(256), 0, st, a));
    return 0;
  }
  if (a.elt == KGE_ELT_F32) {
    KGE_CUDA_OK(launch_pdl(short_conv_kernel<float>, dim3(a.T, cy), dim3(256), 0, st, a));
    KGE_CUDA_OK(launch_pdl(short_conv_save_kernel<float>, dim3(a.B, cb), dim3(256), 0, st, a));
  } else {
    KGE_CUDA_OK(launch_pdl(short_conv_kernel<__nv_bfloat16>, dim3(a.T, cy), dim3(256), 0, st, a));
    KGE_CUDA_OK(launch_pdl(short_conv_save_kernel<__nv_bfloat16>, dim3(a.B, cb), dim3(256), 0, st, a));
  }
  return 0;
}

}  // namespace kge
