// Hyper-connected residual for layer-list models: the residual stream exists in S copies ("streams"), xs [T, S, d] in
// fp32.  A sublayer reads a weighted sum of the streams through an RMS norm, and its result y comes back into every
// stream while the old streams are mixed by an S x S matrix:
//     u = sum_s in[s] x_s,    x_j <- sum_s mix[s, j] x_s + out[j] * (mult * col_scale . y)
// With S = 1, in = out = mix = 1 this is the plain pre-norm residual x <- x + mult * col_scale . y.  One block per
// token; every sum of a row runs in a fixed order in fp32, whatever else the launch holds.
#include "common.cuh"
#include "elt_access.cuh"
#include "hybrid_ops.h"

namespace kge {

constexpr int SMAX = 8;

template <typename E>
__global__ void __launch_bounds__(256) embed_norm_streams_kernel(float* xs, const int32_t* ids, const E* table, const E* norm_w, int d, int S, float eps) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float red[33];
  const int t = blockIdx.x;
  const E* row = table + (int64_t)ids[t] * d;
  float inv = 1.f;
  if (norm_w) {
    float ss = 0.f;
    for (int c = threadIdx.x; c < d; c += blockDim.x) { const float v = ldf(row + c); ss = fmaf(v, v, ss); }
    inv = 1.f / sqrtf(block_sum(ss, red) / (float)d + eps);
  }
  float* x = xs + (int64_t)t * S * d;
  for (int c = threadIdx.x; c < d; c += blockDim.x) {
    const float v = norm_w ? ldf(row + c) * inv * ldf(norm_w + c) : ldf(row + c);
    for (int s = 0; s < S; ++s) x[(int64_t)s * d + c] = v;
  }
}

int embed_norm_streams(float* xs, const int32_t* ids, const void* table, const void* norm_w, int T, int d, int S, float eps, int elt, cudaStream_t st) {
  if (T <= 0) return 0;
  KGE_REQUIRE(S >= 1 && S <= SMAX, "embed_norm_streams: %d streams", S);
  cudaError_t ce = elt == KGE_ELT_F32
      ? launch_pdl(embed_norm_streams_kernel<float>, dim3(T), dim3(256), 0, st, xs, ids, (const float*)table, (const float*)norm_w, d, S, eps)
      : launch_pdl(embed_norm_streams_kernel<__nv_bfloat16>, dim3(T), dim3(256), 0, st, xs, ids, (const __nv_bfloat16*)table, (const __nv_bfloat16*)norm_w, d, S, eps);
  KGE_CUDA_OK(ce);
  return 0;
}

// u is kept in shared memory between the sum of squares and the write (one read of the streams)
template <typename E>
__global__ void __launch_bounds__(256) stream_norm_kernel(StreamNormArgs a) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ float u[];
  __shared__ float red[33];
  __shared__ float win[SMAX];
  const int r = blockIdx.x, row = a.rows ? a.rows[r] : r, d = a.d, S = a.S;
  if (threadIdx.x < S) win[threadIdx.x] = a.in_w ? a.in_w[threadIdx.x] : 1.f;
  __syncthreads();
  const float* x = a.xs + (int64_t)row * S * d;
  float ss = 0.f;
  for (int c = threadIdx.x; c < d; c += blockDim.x) {
    float v = win[0] * x[c];
    for (int s = 1; s < S; ++s) v = fmaf(win[s], x[(int64_t)s * d + c], v);
    u[c] = v;
    ss = fmaf(v, v, ss);
  }
  const float inv = 1.f / sqrtf(block_sum(ss, red) / (float)d + a.eps) * a.out_scale;
  E* y = (E*)a.y + (int64_t)r * d;
  for (int c = threadIdx.x; c < d; c += blockDim.x) {
    const float v = u[c];
    if (a.y) stf(y + c, v * inv * ldf((const E*)a.w + c));
    if (a.sum_out) a.sum_out[(int64_t)r * d + c] = v;
  }
}

// the same arithmetic as stream_norm_kernel, column for column, four columns per thread and pass
template <typename E>
__global__ void __launch_bounds__(256) stream_norm_vec_kernel(StreamNormArgs a) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ __align__(16) float u[];
  __shared__ float red[33];
  __shared__ float win[SMAX];
  const int r = blockIdx.x, row = a.rows ? a.rows[r] : r, d = a.d, S = a.S;
  if (threadIdx.x < S) win[threadIdx.x] = a.in_w ? a.in_w[threadIdx.x] : 1.f;
  __syncthreads();
  const float* x = a.xs + (int64_t)row * S * d;
  float ss = 0.f;
  for (int c = threadIdx.x * 4; c < d; c += blockDim.x * 4) {
    float v[4], t[4];
    ld4(x + c, v);
#pragma unroll
    for (int i = 0; i < 4; ++i) v[i] = win[0] * v[i];
    for (int s = 1; s < S; ++s) {
      ld4(x + (int64_t)s * d + c, t);
#pragma unroll
      for (int i = 0; i < 4; ++i) v[i] = fmaf(win[s], t[i], v[i]);
    }
    st4(u + c, v);
#pragma unroll
    for (int i = 0; i < 4; ++i) ss = fmaf(v[i], v[i], ss);
  }
  const float inv = 1.f / sqrtf(block_sum(ss, red) / (float)d + a.eps) * a.out_scale;
  E* y = (E*)a.y + (int64_t)r * d;
  for (int c = threadIdx.x * 4; c < d; c += blockDim.x * 4) {
    float v[4], w[4];
    ld4(u + c, v);
    if (a.y) {
      ld4((const E*)a.w + c, w);
#pragma unroll
      for (int i = 0; i < 4; ++i) w[i] = v[i] * inv * w[i];
      st4(y + c, w);
    }
    if (a.sum_out) st4(a.sum_out + (int64_t)r * d + c, v);
  }
}

template <typename E>
__global__ void __launch_bounds__(256) stream_combine_vec_kernel(StreamCombineArgs a) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ __align__(16) float un[];
  __shared__ float mix[SMAX * SMAX], wout[SMAX], win[SMAX], rs[4], red[33];
  const int t = blockIdx.x, d = a.d, S = a.S;
  if (threadIdx.x < S) win[threadIdx.x] = a.next_in ? a.next_in[threadIdx.x] : 1.f;
  if (threadIdx.x < S * S) mix[threadIdx.x] = a.mix ? a.mix[threadIdx.x] : (threadIdx.x / S == threadIdx.x % S ? 1.f : 0.f);
  if (threadIdx.x < S) wout[threadIdx.x] = a.out_w ? a.out_w[threadIdx.x] : 1.f;
  if (threadIdx.x < a.src.n) rs[threadIdx.x] = a.src.scale[threadIdx.x] * (a.src.rscale[threadIdx.x] ? a.src.rscale[threadIdx.x][(int64_t)t * a.src.rs_stride[threadIdx.x]] : 1.f);
  __syncthreads();
  float* x = a.xs + (int64_t)t * S * d;
  float ss = 0.f;
  for (int c = threadIdx.x * 4; c < d; c += blockDim.x * 4) {
    float y[4] = {0.f, 0.f, 0.f, 0.f}, q[4];
    if (a.y32) ld4(a.y32 + (int64_t)t * d + c, y);
    for (int i = 0; i < a.src.n; ++i) {
      ld4((const E*)a.src.src[i] + (int64_t)t * a.src.ld[i] + c, q);
#pragma unroll
      for (int k = 0; k < 4; ++k) y[k] = fmaf(rs[i], q[k], y[k]);
    }
    float z[4] = {1.f, 1.f, 1.f, 1.f};
    if (a.col_scale) ld4(a.col_scale + c, z);
#pragma unroll
    for (int k = 0; k < 4; ++k) z[k] = a.mult * z[k] * y[k];
    float old[SMAX][4];
#pragma unroll
    for (int s = 0; s < SMAX; ++s) if (s < S) ld4(x + (int64_t)s * d + c, old[s]);
    float u[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int j = 0; j < SMAX; ++j) {
      if (j < S) {
        float v[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int s = 0; s < SMAX; ++s)
          if (s < S) {
#pragma unroll
            for (int k = 0; k < 4; ++k) v[k] = fmaf(mix[s * S + j], old[s][k], v[k]);
          }
#pragma unroll
        for (int k = 0; k < 4; ++k) { v[k] = fmaf(wout[j], z[k], v[k]); u[k] = j == 0 ? win[0] * v[k] : fmaf(win[j], v[k], u[k]); }
        st4(x + (int64_t)j * d + c, v);
      }
    }
    if (a.next_y) {
      st4(un + c, u);
#pragma unroll
      for (int k = 0; k < 4; ++k) ss = fmaf(u[k], u[k], ss);
    }
  }
  if (!a.next_y) return;
  const float inv = 1.f / sqrtf(block_sum(ss, red) / (float)d + a.eps);
  E* y2 = (E*)a.next_y + (int64_t)t * d;
  for (int c = threadIdx.x * 4; c < d; c += blockDim.x * 4) {
    float v[4], w[4];
    ld4(un + c, v);
    ld4((const E*)a.next_w + c, w);
#pragma unroll
    for (int k = 0; k < 4; ++k) w[k] = v[k] * inv * w[k];
    st4(y2 + c, w);
  }
}

static bool al16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

int stream_norm(const StreamNormArgs& a, cudaStream_t st) {
  if (a.R <= 0) return 0;
  KGE_REQUIRE(a.S >= 1 && a.S <= SMAX && a.d > 0 && (size_t)a.d * 4 <= 200 * 1024, "stream_norm: %d streams of %d columns", a.S, a.d);
  const size_t smem = (size_t)a.d * 4;
  static size_t smem_set = 0;
  if (smem > 48 * 1024 && smem > smem_set) {
    KGE_CUDA_OK(cudaFuncSetAttribute(stream_norm_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    KGE_CUDA_OK(cudaFuncSetAttribute(stream_norm_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  }
  const bool vec = a.d % 8 == 0 && al16(a.xs) && al16(a.y) && al16(a.w) && al16(a.sum_out);
  if (vec && smem > 48 * 1024 && smem > smem_set) {
    KGE_CUDA_OK(cudaFuncSetAttribute(stream_norm_vec_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    KGE_CUDA_OK(cudaFuncSetAttribute(stream_norm_vec_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  }
  if (smem > 48 * 1024 && smem > smem_set) smem_set = smem;
  cudaError_t ce;
  if (vec) ce = a.elt == KGE_ELT_F32 ? launch_pdl(stream_norm_vec_kernel<float>, dim3(a.R), dim3(256), smem, st, a)
                                     : launch_pdl(stream_norm_vec_kernel<__nv_bfloat16>, dim3(a.R), dim3(256), smem, st, a);
  else ce = a.elt == KGE_ELT_F32 ? launch_pdl(stream_norm_kernel<float>, dim3(a.R), dim3(256), smem, st, a)
                                 : launch_pdl(stream_norm_kernel<__nv_bfloat16>, dim3(a.R), dim3(256), smem, st, a);
  KGE_CUDA_OK(ce);
  return 0;
}

template <typename E>
__global__ void __launch_bounds__(256) stream_combine_kernel(StreamCombineArgs a) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ float un[];                  // the next sublayer's input row before its norm (only with next_y)
  __shared__ float mix[SMAX * SMAX], wout[SMAX], win[SMAX], rs[4], red[33];
  const int t = blockIdx.x, d = a.d, S = a.S;
  if (threadIdx.x < S) win[threadIdx.x] = a.next_in ? a.next_in[threadIdx.x] : 1.f;
  if (threadIdx.x < S * S) mix[threadIdx.x] = a.mix ? a.mix[threadIdx.x] : (threadIdx.x / S == threadIdx.x % S ? 1.f : 0.f);
  if (threadIdx.x < S) wout[threadIdx.x] = a.out_w ? a.out_w[threadIdx.x] : 1.f;
  if (threadIdx.x < a.src.n) rs[threadIdx.x] = a.src.scale[threadIdx.x] * (a.src.rscale[threadIdx.x] ? a.src.rscale[threadIdx.x][(int64_t)t * a.src.rs_stride[threadIdx.x]] : 1.f);
  __syncthreads();
  float* x = a.xs + (int64_t)t * S * d;
  float ss = 0.f;
  for (int c = threadIdx.x; c < d; c += blockDim.x) {
    float y = a.y32 ? a.y32[(int64_t)t * d + c] : 0.f;
    for (int i = 0; i < a.src.n; ++i) y = fmaf(rs[i], ldf((const E*)a.src.src[i] + (int64_t)t * a.src.ld[i] + c), y);
    const float z = a.mult * (a.col_scale ? a.col_scale[c] : 1.f) * y;
    float old[SMAX];
#pragma unroll
    for (int s = 0; s < SMAX; ++s) old[s] = s < S ? x[(int64_t)s * d + c] : 0.f;
    float u = 0.f;
#pragma unroll
    for (int j = 0; j < SMAX; ++j) {
      if (j < S) {
        float v = 0.f;
#pragma unroll
        for (int s = 0; s < SMAX; ++s) if (s < S) v = fmaf(mix[s * S + j], old[s], v);
        v = fmaf(wout[j], z, v);
        x[(int64_t)j * d + c] = v;
        u = j == 0 ? win[0] * v : fmaf(win[j], v, u);      // the same order of summation as stream_norm
      }
    }
    if (a.next_y) { un[c] = u; ss = fmaf(u, u, ss); }
  }
  if (!a.next_y) return;
  const float inv = 1.f / sqrtf(block_sum(ss, red) / (float)d + a.eps);
  E* y2 = (E*)a.next_y + (int64_t)t * d;
  for (int c = threadIdx.x; c < d; c += blockDim.x) stf(y2 + c, un[c] * inv * ldf((const E*)a.next_w + c));
}

int stream_combine(const StreamCombineArgs& a, cudaStream_t st) {
  if (a.T <= 0) return 0;
  KGE_REQUIRE(a.S >= 1 && a.S <= SMAX && a.src.n >= 0 && a.src.n <= 4, "stream_combine: %d streams, %d sources", a.S, a.src.n);
  const size_t smem = a.next_y ? (size_t)a.d * 4 : 0;
  KGE_REQUIRE(smem <= 200 * 1024, "stream_combine: rows of %d columns", a.d);
  static size_t smem_set = 0;
  if (smem > 48 * 1024 && smem > smem_set) {
    KGE_CUDA_OK(cudaFuncSetAttribute(stream_combine_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    KGE_CUDA_OK(cudaFuncSetAttribute(stream_combine_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  }
  bool vec = a.d % 8 == 0 && al16(a.xs) && al16(a.y32) && al16(a.col_scale) && al16(a.next_y) && al16(a.next_w);
  for (int i = 0; i < a.src.n; ++i) vec = vec && al16(a.src.src[i]) && a.src.ld[i] % 8 == 0;
  if (vec && smem > 48 * 1024 && smem > smem_set) {
    KGE_CUDA_OK(cudaFuncSetAttribute(stream_combine_vec_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    KGE_CUDA_OK(cudaFuncSetAttribute(stream_combine_vec_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  }
  if (smem > 48 * 1024 && smem > smem_set) smem_set = smem;
  cudaError_t ce;
  if (vec) ce = a.elt == KGE_ELT_F32 ? launch_pdl(stream_combine_vec_kernel<float>, dim3(a.T), dim3(256), smem, st, a)
                                     : launch_pdl(stream_combine_vec_kernel<__nv_bfloat16>, dim3(a.T), dim3(256), smem, st, a);
  else ce = a.elt == KGE_ELT_F32 ? launch_pdl(stream_combine_kernel<float>, dim3(a.T), dim3(256), smem, st, a)
                                 : launch_pdl(stream_combine_kernel<__nv_bfloat16>, dim3(a.T), dim3(256), smem, st, a);
  KGE_CUDA_OK(ce);
  return 0;
}

}  // namespace kge
