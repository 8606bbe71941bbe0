// RMS norms in groups for layer-list models that norm a sublayer's input AND its result: the row is cut into `groups`
// equal consecutive parts, each divided by its own root mean square.  One block per row; the row stays in shared memory
// (fp32) between the statistics and the write, so the residual stream is read once and written once per sublayer, and the
// pass that adds a sublayer's result also forms the next sublayer's normed input.  Every sum of a row is formed in a
// fixed order that depends on the row's width only, never on what else is in the launch.
#include "common.cuh"
#include "elt_access.cuh"
#include "hybrid_ops.h"

namespace kge {

namespace {

constexpr int GN_THREADS = 256, GN_MAX_GROUPS = 1024;

// sum of squares of every group of a shared row: warp w takes groups w, w + nwarps, ..; the result is the factor
// 1 / sqrt(mean + eps) per group in inv[]
__device__ __forceinline__ void group_inv_rms(const float* row, int d, int groups, float eps, float* inv) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5, gs = d / groups;
  for (int g = warp; g < groups; g += nw) {
    float ss = 0.f;
    for (int c = lane; c < gs; c += 32) { const float v = row[g * gs + c]; ss = fmaf(v, v, ss); }
    ss = warp_sum(ss);
    if (lane == 0) inv[g] = 1.f / sqrtf(ss / (float)gs + eps);
  }
}

template <typename E>
__global__ void __launch_bounds__(GN_THREADS) group_rmsnorm_kernel(E* y, const float* x, const int32_t* rows, const E* w, int d, int groups, float eps, float out_scale) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ __align__(16) float gn_sm[];
  float* row = gn_sm;
  __shared__ float inv[GN_MAX_GROUPS];
  const int r = blockIdx.x;
  const float* src = x + (int64_t)(rows ? rows[r] : r) * d;
  for (int c = threadIdx.x; c < d; c += GN_THREADS) row[c] = src[c];
  __syncthreads();
  group_inv_rms(row, d, groups, eps, inv);
  __syncthreads();
  const int gs = d / groups;
  for (int c = threadIdx.x; c < d; c += GN_THREADS) stf(y + (int64_t)r * d + c, row[c] * inv[c / gs] * ldf(w + c) * out_scale);
}

// VEC: four neighbouring columns per thread and pass (rows and groups of 4-column multiples, 16-byte aligned): 8-byte
// loads of 16-bit rows, 16-byte ones of fp32 rows; the sums are formed in the same order either way
template <typename E, bool VEC>
__global__ void __launch_bounds__(GN_THREADS) postnorm_residual_kernel(PostNormArgs a) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ __align__(16) float gn_sm[];
  const int d = a.d, t = blockIdx.x, gs = d / a.groups;
  constexpr int W = VEC ? 4 : 1;
  float* ya = gn_sm;                 // the sublayer's result, then the new residual row
  float* yb = gn_sm + d;             // the second source
  __shared__ float inv[GN_MAX_GROUPS], red[33];
  float f[2] = {1.f, 1.f};
  for (int i = 0; i < a.nsrc; ++i) {
    const E* s = (const E*)a.src[i] + (int64_t)t * a.ld[i];
    float* dst = i ? yb : ya;
    float ss = 0.f;
    for (int c = threadIdx.x * W; c < d; c += GN_THREADS * W) {
      float v[4];
      if (VEC) ld4(s + c, v); else v[0] = ldf(s + c);
#pragma unroll
      for (int k = 0; k < W; ++k) { dst[c + k] = v[k]; ss = fmaf(v[k], v[k], ss); }
    }
    if (a.inner_w[i]) f[i] = 1.f / sqrtf(block_sum(ss, red) / (float)d + a.eps);
  }
  __syncthreads();
  for (int c = threadIdx.x * W; c < d; c += GN_THREADS * W) {
    float w0[4] = {1.f, 1.f, 1.f, 1.f}, w1[4] = {1.f, 1.f, 1.f, 1.f};
    if (a.inner_w[0]) { if (VEC) ld4((const E*)a.inner_w[0] + c, w0); else w0[0] = ldf((const E*)a.inner_w[0] + c); }
    if (a.nsrc > 1 && a.inner_w[1]) { if (VEC) ld4((const E*)a.inner_w[1] + c, w1); else w1[0] = ldf((const E*)a.inner_w[1] + c); }
#pragma unroll
    for (int k = 0; k < W; ++k) {
      float v = a.inner_w[0] ? ya[c + k] * f[0] * w0[k] : ya[c + k];
      if (a.nsrc > 1) v += a.inner_w[1] ? yb[c + k] * f[1] * w1[k] : yb[c + k];
      ya[c + k] = v * a.src_scale;
    }
  }
  __syncthreads();
  group_inv_rms(ya, d, a.groups, a.eps, inv);
  __syncthreads();
  float* res = a.res + (int64_t)t * d;
  for (int c = threadIdx.x * W; c < d; c += GN_THREADS * W) {
    float r[4], w[4];
    if (VEC) { ld4(res + c, r); ld4((const E*)a.post_w + c, w); } else { r[0] = res[c]; w[0] = ldf((const E*)a.post_w + c); }
    const float gi = inv[c / gs];
#pragma unroll
    for (int k = 0; k < W; ++k) { r[k] += ya[c + k] * gi * w[k]; ya[c + k] = r[k]; }
    if (VEC) st4(res + c, r); else res[c] = r[0];
  }
  if (!a.next_w) return;
  __syncthreads();
  group_inv_rms(ya, d, a.groups, a.eps, inv);
  __syncthreads();
  E* ny = (E*)a.next_y + (int64_t)t * d;
  for (int c = threadIdx.x * W; c < d; c += GN_THREADS * W) {
    float w[4], o[4];
    if (VEC) ld4((const E*)a.next_w + c, w); else w[0] = ldf((const E*)a.next_w + c);
    const float gi = inv[c / gs];
#pragma unroll
    for (int k = 0; k < W; ++k) o[k] = ya[c + k] * gi * w[k];
    if (VEC) st4(ny + c, o); else stf(ny + c, o[0]);
  }
}

template <typename E>
__global__ void __launch_bounds__(256) silu_mul_halves_kernel(E* y, const E* gu, int64_t n, int f) {
  pdl_launch_dependents();
  pdl_wait();
  const int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x;
  if (i >= n) return;
  const int64_t t = i / f, c = i % f;
  const float g = ldf(gu + t * 2 * f + c), u = ldf(gu + t * 2 * f + f + c);
  stf(y + i, g / (1.f + expf(-g)) * u);
}

template <typename K>
int opt_in_smem(K kern, size_t smem) {
  if (smem > 48 * 1024) KGE_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  return 0;
}

}  // namespace

int group_rmsnorm_f32in(void* y, const float* x, const int32_t* rows, const void* w, int R, int d, int groups, float eps, float out_scale, int elt,
                        cudaStream_t st) {
  if (R <= 0) return 0;
  KGE_REQUIRE(groups >= 1 && groups <= GN_MAX_GROUPS && d % groups == 0 && d <= 51200, "group_rmsnorm: %d groups of a row of %d", groups, d);
  const size_t smem = (size_t)d * 4;
  if (elt == KGE_ELT_F32) {
    if (int rc = opt_in_smem(group_rmsnorm_kernel<float>, smem)) return rc;
    KGE_CUDA_OK(launch_pdl(group_rmsnorm_kernel<float>, dim3(R), dim3(GN_THREADS), smem, st, (float*)y, x, rows, (const float*)w, d, groups, eps, out_scale));
  } else {
    if (int rc = opt_in_smem(group_rmsnorm_kernel<__nv_bfloat16>, smem)) return rc;
    KGE_CUDA_OK(launch_pdl(group_rmsnorm_kernel<__nv_bfloat16>, dim3(R), dim3(GN_THREADS), smem, st, (__nv_bfloat16*)y, x, rows, (const __nv_bfloat16*)w, d, groups, eps, out_scale));
  }
  return 0;
}

int postnorm_residual(const PostNormArgs& a, cudaStream_t st) {
  if (a.T <= 0) return 0;
  KGE_REQUIRE(a.groups >= 1 && a.groups <= GN_MAX_GROUPS && a.d % a.groups == 0 && a.d <= 25600 && a.nsrc >= 1 && a.nsrc <= 2 && a.post_w,
              "postnorm_residual: %d groups of a row of %d, %d sources", a.groups, a.d, a.nsrc);
  const size_t smem = (size_t)a.d * 8;
  bool vec = a.d % 4 == 0 && (a.d / a.groups) % 4 == 0 && ((uintptr_t)a.res & 15) == 0 && ((uintptr_t)a.post_w & 15) == 0 &&
             (!a.next_w || ((((uintptr_t)a.next_w | (uintptr_t)a.next_y) & 15) == 0));
  for (int i = 0; i < a.nsrc; ++i) vec = vec && a.ld[i] % 4 == 0 && ((uintptr_t)a.src[i] & 15) == 0 && (!a.inner_w[i] || ((uintptr_t)a.inner_w[i] & 15) == 0);
  if (a.elt == KGE_ELT_F32) {
    if (int rc = opt_in_smem(postnorm_residual_kernel<float, false>, smem)) return rc;
    if (int rc = opt_in_smem(postnorm_residual_kernel<float, true>, smem)) return rc;
    KGE_CUDA_OK(vec ? launch_pdl(postnorm_residual_kernel<float, true>, dim3(a.T), dim3(GN_THREADS), smem, st, a)
                    : launch_pdl(postnorm_residual_kernel<float, false>, dim3(a.T), dim3(GN_THREADS), smem, st, a));
  } else {
    if (int rc = opt_in_smem(postnorm_residual_kernel<__nv_bfloat16, false>, smem)) return rc;
    if (int rc = opt_in_smem(postnorm_residual_kernel<__nv_bfloat16, true>, smem)) return rc;
    KGE_CUDA_OK(vec ? launch_pdl(postnorm_residual_kernel<__nv_bfloat16, true>, dim3(a.T), dim3(GN_THREADS), smem, st, a)
                    : launch_pdl(postnorm_residual_kernel<__nv_bfloat16, false>, dim3(a.T), dim3(GN_THREADS), smem, st, a));
  }
  return 0;
}

int silu_mul_halves(void* y, const void* gu, int T, int f, int elt, cudaStream_t st) {
  const int64_t n = (int64_t)T * f;
  if (n <= 0) return 0;
  const dim3 grid((unsigned)((n + 255) / 256));
  if (elt == KGE_ELT_F32) KGE_CUDA_OK(launch_pdl(silu_mul_halves_kernel<float>, grid, dim3(256), 0, st, (float*)y, (const float*)gu, n, f));
  else KGE_CUDA_OK(launch_pdl(silu_mul_halves_kernel<__nv_bfloat16>, grid, dim3(256), 0, st, (__nv_bfloat16*)y, (const __nv_bfloat16*)gu, n, f));
  return 0;
}

}  // namespace kge
