// A short causal convolution over time on every channel of a projection, continued across steps from a state slot that
// holds the request's last taps - 1 input rows.  Each output is a sum over the taps in ascending order in fp32, from
// this step's rows or the slot's, so the result does not depend on where a prompt was cut.
#include "common.cuh"
#include "elt_access.cuh"
#include "hybrid_ops.h"

namespace kge {

namespace {

constexpr int SC_MAX_TAPS = 16;

// one block per token; a thread walks channels
template <typename E>
__global__ void __launch_bounds__(256) short_conv_kernel(ShortConvArgs a) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x, b = a.token_req[t], r0 = a.qsl[b], pos = a.positions[t], taps = a.taps;
  const float* sp = a.state + (int64_t)a.slots[b] * a.slot_stride;      // [taps - 1, C]: row s holds the input of position p0 - (taps - 1) + s
  const E* x = (const E*)a.x;
  for (int c = threadIdx.x; c < a.C; c += blockDim.x) {
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

// one block per request: the slot's rows move up by the step's row count and the step's last rows follow
template <typename E>
__global__ void __launch_bounds__(256) short_conv_save_kernel(ShortConvArgs a) {
  pdl_launch_dependents();
  pdl_wait();
  const int b = blockIdx.x, r0 = a.qsl[b], n = a.qsl[b + 1] - r0, keep = a.taps - 1;
  if (n <= 0 || keep <= 0) return;
  const bool fresh = a.positions[r0] == 0;
  float* sp = a.state + (int64_t)a.slots[b] * a.slot_stride;
  const E* x = (const E*)a.x;
  for (int c = threadIdx.x; c < a.C; c += blockDim.x) {
    for (int s = 0; s < keep; ++s) {                  // ascending: row s only reads rows above it
      const int src = s + n;                          // in the old numbering of the slot's rows
      float v;
      if (src >= keep) v = ldf(x + (int64_t)(r0 + src - keep) * a.ldx + c);
      else v = fresh ? 0.f : sp[(int64_t)src * a.C + c];
      sp[(int64_t)s * a.C + c] = v;
    }
  }
}

}  // namespace

int short_conv_state(const ShortConvArgs& a, cudaStream_t st) {
  if (a.T <= 0) return 0;
  KGE_REQUIRE(a.taps >= 1 && a.taps <= SC_MAX_TAPS && a.C > 0 && a.x != a.y, "short_conv_state: %d taps on %d channels", a.taps, a.C);
  if (a.elt == KGE_ELT_F32) {
    KGE_CUDA_OK(launch_pdl(short_conv_kernel<float>, dim3(a.T), dim3(256), 0, st, a));
    KGE_CUDA_OK(launch_pdl(short_conv_save_kernel<float>, dim3(a.B), dim3(256), 0, st, a));
  } else {
    KGE_CUDA_OK(launch_pdl(short_conv_kernel<__nv_bfloat16>, dim3(a.T), dim3(256), 0, st, a));
    KGE_CUDA_OK(launch_pdl(short_conv_save_kernel<__nv_bfloat16>, dim3(a.B), dim3(256), 0, st, a));
  }
  return 0;
}

}  // namespace kge
