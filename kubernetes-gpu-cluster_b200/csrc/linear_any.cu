// Shape-agnostic linear layer for layer-list models: any T / N / K and alignment, bfloat16 or float32 storage, fp32
// accumulation in a fixed k order (so a row's result does not depend on what else is in the launch), optional row
// gather / scatter, per-row input scale, grouped rows (one weight slice per group: mixture-of-experts) or strided slices
// (block-diagonal projections), gated pairs (silu(x.w) * (x.w2)) and fp32 output or accumulation.  Tiles of 64 x 64
// outputs and 256 threads: float32 storage multiplies on the fp32 pipes (4 x 4 outputs per thread, operands staged in
// shared memory as fp32, true 32-bit products), bfloat16 storage on the tensor cores (mma.sync, further down).
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <algorithm>

#include "common.cuh"
#include "elt_access.cuh"
#include "hybrid_ops.h"

namespace kge {

__device__ __forceinline__ float act_apply(int act, float v) {
  switch (act) {
    case ACT_GELU_ERF: return 0.5f * v * (1.f + erff(v * 0.70710678118654752f));
    case ACT_GELU_TANH: return 0.5f * v * (1.f + tanhf(0.79788456080286536f * (v + 0.044715f * v * v * v)));
    case ACT_SILU: return v / (1.f + expf(-v));
    case ACT_SIGMOID: return 1.f / (1.f + expf(-v));
    case ACT_TANH: return tanhf(v);
    case ACT_RELU2: { const float r = fmaxf(v, 0.f); return r * r; }
    default: return v;
  }
}

// the gated pair of two pre-activations (row scale applied)
__device__ __forceinline__ float glu_apply(const LinearArgs& a, float g, float u) {
  if (a.glu == GLU_CLAMPED_SIGMOID) {
    g = fminf(g, a.glu_limit);
    u = fminf(fmaxf(u, -a.glu_limit), a.glu_limit);
    return g / (1.f + expf(-a.glu_alpha * g)) * (u + 1.f);
  }
  return act_apply(ACT_SILU, g) * u;
}

constexpr int LBM = 64, LBN = 64, LBK = 16;

template <typename E, typename O, bool DUAL>
__global__ void __launch_bounds__(256) linear_any_kernel(LinearArgs a) {
  pdl_launch_dependents();
  pdl_wait();
  const int z = blockIdx.z;
  int r0 = 0, r1 = a.T;
  if (a.group_off) { r0 = a.group_off[z]; r1 = a.group_off[z + 1]; }
  const int m0 = r0 + blockIdx.y * LBM;
  if (m0 >= r1) return;
  const int n0 = blockIdx.x * LBN;
  const E* x = (const E*)a.x + z * a.x_zs;
  const E* w = (const E*)a.w + z * a.w_zs;
  const E* w2 = DUAL ? (const E*)a.w2 + z * a.w_zs : nullptr;
  const E* bias = a.bias ? (const E*)a.bias + z * a.b_zs : nullptr;
  O* y = (O*)a.y + z * a.y_zs;
  __shared__ float xs[LBK][LBM + 1], ws[LBK][LBN + 1], ws2[DUAL ? LBK : 1][LBN + 1];
  __shared__ int xrow[LBM];
  const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
  if (tid < LBM) {
    const int r = m0 + tid;
    xrow[tid] = r < r1 ? (a.xrows ? a.xrows[r] : r) : -1;
  }
  __syncthreads();
  float acc[4][4] = {}, acc2[DUAL ? 4 : 1][4] = {};
  for (int k0 = 0; k0 < a.K; k0 += LBK) {
    for (int i = tid; i < LBM * LBK; i += 256) {
      const int r = i / LBK, k = i % LBK;
      const int xr = xrow[r];
      xs[k][r] = (xr >= 0 && k0 + k < a.K) ? ldf(x + (int64_t)xr * a.ldx + k0 + k) : 0.f;
      const int n = n0 + r;
      const bool ok = n < a.N && k0 + k < a.K;
      ws[k][r] = ok ? ldf(w + (int64_t)n * a.K + k0 + k) : 0.f;
      if (DUAL) ws2[k][r] = ok ? ldf(w2 + (int64_t)n * a.K + k0 + k) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < LBK; ++k) {
      float xv[4], wv[4], wv2[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) { xv[i] = xs[k][ty * 4 + i]; wv[i] = ws[k][tx * 4 + i]; if (DUAL) wv2[i] = ws2[k][tx * 4 + i]; }
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          acc[i][j] = fmaf(xv[i], wv[j], acc[i][j]);
          if (DUAL) acc2[i][j] = fmaf(xv[i], wv2[j], acc2[i][j]);
        }
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int r = m0 + ty * 4 + i;
    if (r >= r1) continue;
    const float s = a.row_scale ? a.row_scale[r] : 1.f;
    const int yr = a.yrows ? a.yrows[r] : r;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      if (n >= a.N) continue;
      float v;
      if (DUAL) v = glu_apply(a, s * acc[i][j], s * acc2[i][j]);
      else v = act_apply(a.act, s * acc[i][j] + (bias ? ldf(bias + n) : 0.f));
      v *= a.alpha;
      O* dst = y + (int64_t)yr * a.ldy + n;
      if (a.accumulate) v += ldf(dst);
      stf(dst, v);
    }
  }
}

// bfloat16 operands: the same tiling on the tensor cores (mma.sync m16n8k16, fp32 accumulators).  Both operands are
// k-contiguous, which is exactly the row x col fragment layout, so the fragments are 32-bit loads from k-padded shared
// tiles.  Eight warps as 2 x 4, each 32 rows x 16 outputs; a row's sum is formed in the same k order whatever the launch holds.
constexpr int MPAD = 8;       // the k-tile is 32 wide for many rows and 64 for few (weight streaming: fewer, fatter round trips)

__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// eight consecutive k of one row as one 16-byte register, zero beyond K or for a missing row; one 16-byte load when aligned
__device__ __forceinline__ uint4 load8(const __nv_bfloat16* row, int k, int K, bool vec) {
  if (row && vec && k + 8 <= K) return *reinterpret_cast<const uint4*>(row + k);
  union { uint4 v; __nv_bfloat16 e[8]; } u;
#pragma unroll
  for (int i = 0; i < 8; ++i) u.e[i] = (row && k + i < K) ? row[k + i] : __float2bfloat16_rn(0.f);
  return u.v;
}

template <typename O, bool DUAL, int MBK>
__global__ void __launch_bounds__(256) linear_mma_kernel(LinearArgs a) {
  pdl_launch_dependents();
  pdl_wait();
  typedef __nv_bfloat16 E;
  const int z = blockIdx.z;
  int r0 = 0, r1 = a.T;
  if (a.group_off) { r0 = a.group_off[z]; r1 = a.group_off[z + 1]; }
  const int m0 = r0 + blockIdx.y * LBM;
  if (m0 >= r1) return;
  const int n0 = blockIdx.x * LBN;
  const E* x = (const E*)a.x + z * a.x_zs;
  const E* w = (const E*)a.w + z * a.w_zs;
  const E* w2 = DUAL ? (const E*)a.w2 + z * a.w_zs : nullptr;
  const E* bias = a.bias ? (const E*)a.bias + z * a.b_zs : nullptr;
  O* y = (O*)a.y + z * a.y_zs;
  __shared__ __align__(16) E xs[LBM][MBK + MPAD], ws[LBN][MBK + MPAD], ws2[DUAL ? LBN : 1][MBK + MPAD];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int wm = (warp >> 2) * 32, wn = (warp & 3) * 16;
  // staging: thread -> (row tid / 4, eight k at (tid % 4) * 8)
  const int sr = tid >> 2, sk = (tid & 3) * 8;
  const int gr = m0 + sr;
  const E* xrow = gr < r1 ? x + (int64_t)(a.xrows ? a.xrows[gr] : gr) * a.ldx : nullptr;
  const E* wrow = n0 + sr < a.N ? w + (int64_t)(n0 + sr) * a.K : nullptr;
  const E* w2row = (DUAL && n0 + sr < a.N) ? w2 + (int64_t)(n0 + sr) * a.K : nullptr;
  const bool xvec = ((reinterpret_cast<uintptr_t>(x) & 15) == 0) && a.ldx % 8 == 0;
  const bool wvec = ((reinterpret_cast<uintptr_t>(w) & 15) == 0) && a.K % 8 == 0 && (!DUAL || (reinterpret_cast<uintptr_t>(w2) & 15) == 0);
  float acc[2][2][4] = {}, acc2[DUAL ? 2 : 1][2][4] = {};
  // the next k-tile travels from global memory to registers while the tensor cores work on the current one
  constexpr int NU = MBK / 32;                 // 16-byte pieces per thread, operand and k-tile
  uint4 px[NU], pw[NU], pw2[NU];
#pragma unroll
  for (int u = 0; u < NU; ++u) {
    px[u] = load8(xrow, sk + u * 32, a.K, xvec);
    pw[u] = load8(wrow, sk + u * 32, a.K, wvec);
    pw2[u] = DUAL ? load8(w2row, sk + u * 32, a.K, wvec) : make_uint4(0u, 0u, 0u, 0u);
  }
  for (int k0 = 0; k0 < a.K; k0 += MBK) {
#pragma unroll
    for (int u = 0; u < NU; ++u) {
      *reinterpret_cast<uint4*>(&xs[sr][sk + u * 32]) = px[u];
      *reinterpret_cast<uint4*>(&ws[sr][sk + u * 32]) = pw[u];
      if (DUAL) *reinterpret_cast<uint4*>(&ws2[sr][sk + u * 32]) = pw2[u];
    }
    __syncthreads();
    if (k0 + MBK < a.K) {
#pragma unroll
      for (int u = 0; u < NU; ++u) {
        px[u] = load8(xrow, k0 + MBK + sk + u * 32, a.K, xvec);
        pw[u] = load8(wrow, k0 + MBK + sk + u * 32, a.K, wvec);
        if (DUAL) pw2[u] = load8(w2row, k0 + MBK + sk + u * 32, a.K, wvec);
      }
    }
#pragma unroll
    for (int ks = 0; ks < MBK / 16; ++ks) {
      const int kc = ks * 16 + (lane & 3) * 2;
      uint32_t af[2][4];
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        const int r = wm + i * 16 + (lane >> 2);
        af[i][0] = *reinterpret_cast<const uint32_t*>(&xs[r][kc]);
        af[i][1] = *reinterpret_cast<const uint32_t*>(&xs[r + 8][kc]);
        af[i][2] = *reinterpret_cast<const uint32_t*>(&xs[r][kc + 8]);
        af[i][3] = *reinterpret_cast<const uint32_t*>(&xs[r + 8][kc + 8]);
      }
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const int n = wn + j * 8 + (lane >> 2);
        const uint32_t b0 = *reinterpret_cast<const uint32_t*>(&ws[n][kc]), b1 = *reinterpret_cast<const uint32_t*>(&ws[n][kc + 8]);
#pragma unroll
        for (int i = 0; i < 2; ++i) mma_bf16_16816(acc[i][j], af[i], b0, b1);
        if (DUAL) {
          const uint32_t c0 = *reinterpret_cast<const uint32_t*>(&ws2[n][kc]), c1 = *reinterpret_cast<const uint32_t*>(&ws2[n][kc + 8]);
#pragma unroll
          for (int i = 0; i < 2; ++i) mma_bf16_16816(acc2[i][j], af[i], c0, c1);
        }
      }
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 2; ++i)
#pragma unroll
    for (int hh = 0; hh < 2; ++hh) {
      const int r = m0 + wm + i * 16 + (lane >> 2) + hh * 8;
      if (r >= r1) continue;
      const float sc = a.row_scale ? a.row_scale[r] : 1.f;
      const int yr = a.yrows ? a.yrows[r] : r;
#pragma unroll
      for (int j = 0; j < 2; ++j)
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          const int n = n0 + wn + j * 8 + (lane & 3) * 2 + c;
          if (n >= a.N) continue;
          const float s1 = acc[i][j][hh * 2 + c];
          float v;
          if (DUAL) v = glu_apply(a, sc * s1, sc * acc2[i][j][hh * 2 + c]);
          else v = act_apply(a.act, sc * s1 + (bias ? ldf(bias + n) : 0.f));
          v *= a.alpha;
          O* dst = y + (int64_t)yr * a.ldy + n;
          if (a.accumulate) v += ldf(dst);
          stf(dst, v);
        }
    }
}

int linear_any(const LinearArgs& a, cudaStream_t st) {
  KGE_REQUIRE(a.x && a.w && a.y && a.N > 0 && a.K > 0 && a.nz > 0, "linear_any: bad arguments");
  if (a.T <= 0) return 0;
  const int rows = a.group_off ? (a.max_rows > 0 ? a.max_rows : a.T) : a.T;
  dim3 grid((a.N + LBN - 1) / LBN, (rows + LBM - 1) / LBM, a.nz), block(256);
  KGE_REQUIRE(grid.y <= 65535 && grid.z <= 65535, "linear_any: too many row tiles (%u) or slices (%u)", grid.y, grid.z);
  cudaError_t ce;
  const bool f32 = a.elt == KGE_ELT_F32;
  KGE_REQUIRE(!f32 || a.out_f32, "linear_any: float32 storage writes float32");
  if (f32) ce = a.w2 ? launch_pdl(linear_any_kernel<float, float, true>, grid, block, 0, st, a) : launch_pdl(linear_any_kernel<float, float, false>, grid, block, 0, st, a);
  else if (a.T <= 256) {       // few rows: the weights are the traffic
    if (a.out_f32) ce = a.w2 ? launch_pdl(linear_mma_kernel<float, true, 64>, grid, block, 0, st, a) : launch_pdl(linear_mma_kernel<float, false, 64>, grid, block, 0, st, a);
    else ce = a.w2 ? launch_pdl(linear_mma_kernel<__nv_bfloat16, true, 64>, grid, block, 0, st, a) : launch_pdl(linear_mma_kernel<__nv_bfloat16, false, 64>, grid, block, 0, st, a);
  } else if (a.out_f32) ce = a.w2 ? launch_pdl(linear_mma_kernel<float, true, 32>, grid, block, 0, st, a) : launch_pdl(linear_mma_kernel<float, false, 32>, grid, block, 0, st, a);
  else ce = a.w2 ? launch_pdl(linear_mma_kernel<__nv_bfloat16, true, 32>, grid, block, 0, st, a) : launch_pdl(linear_mma_kernel<__nv_bfloat16, false, 32>, grid, block, 0, st, a);
  KGE_CUDA_OK(ce);
  return 0;
}

// ------------------------------------------------------------------------------------------------ small row kernels
template <typename E>
__global__ void embed_f32_kernel(float* res, const int32_t* ids, const E* table, int d) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const E* src = table + (int64_t)ids[t] * d;
  for (int c = threadIdx.x; c < d; c += blockDim.x) res[(int64_t)t * d + c] = ldf(src + c);
}
int embed_f32(float* res, const int32_t* ids, const void* table, int T, int d, int elt, cudaStream_t st) {
  if (T <= 0) return 0;
  cudaError_t ce = elt == KGE_ELT_F32 ? launch_pdl(embed_f32_kernel<float>, dim3(T), dim3(128), 0, st, res, ids, (const float*)table, d)
                                      : launch_pdl(embed_f32_kernel<__nv_bfloat16>, dim3(T), dim3(128), 0, st, res, ids, (const __nv_bfloat16*)table, d);
  KGE_CUDA_OK(ce);
  return 0;
}

template <bool LN>      // rows of up to 8192 columns held in registers (defined with the layer norm below)
static bool norm_vec(void* y, const float* x, const int32_t* rows, const void* w, int R, int d, float eps, float offset, float out_scale, int elt, cudaStream_t st,
                     cudaError_t* ce);

template <typename E>
__global__ void rmsnorm_f32in_kernel(E* y, const float* x, const int32_t* rows, const E* w, int d, float eps, float offset, float out_scale) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float red[33];
  const int r = blockIdx.x;
  const float* src = x + (int64_t)(rows ? rows[r] : r) * d;
  float ss = 0.f;
  for (int c = threadIdx.x; c < d; c += blockDim.x) { const float v = src[c]; ss = fmaf(v, v, ss); }
  ss = block_sum(ss, red);
  const float inv = out_scale / sqrtf(ss / (float)d + eps);
  for (int c = threadIdx.x; c < d; c += blockDim.x) stf(y + (int64_t)r * d + c, src[c] * inv * (offset + ldf(w + c)));
}
int rmsnorm_f32in(void* y, const float* x, const int32_t* rows, const void* w, int R, int d, float eps, float offset, float out_scale, int elt,
                  cudaStream_t st) {
  if (R <= 0) return 0;
  cudaError_t ce;
  if (norm_vec<false>(y, x, rows, w, R, d, eps, offset, out_scale, elt, st, &ce)) { KGE_CUDA_OK(ce); return 0; }
  ce = elt == KGE_ELT_F32
      ? launch_pdl(rmsnorm_f32in_kernel<float>, dim3(R), dim3(256), 0, st, (float*)y, x, rows, (const float*)w, d, eps, offset, out_scale)
      : launch_pdl(rmsnorm_f32in_kernel<__nv_bfloat16>, dim3(R), dim3(256), 0, st, (__nv_bfloat16*)y, x, rows, (const __nv_bfloat16*)w, d, eps, offset, out_scale);
  KGE_CUDA_OK(ce);
  return 0;
}

// Both norms for rows of up to 8192 columns (a multiple of 4): the row is read once, as float4, and stays in registers for
// the statistics (layer norm: mean first, then the squared deviations) and the output (four values per store).
constexpr int NV_MAX = 8;
__device__ __forceinline__ float4 ldw4(const float* w) { return *reinterpret_cast<const float4*>(w); }
__device__ __forceinline__ float4 ldw4(const __nv_bfloat16* w) {
  const uint2 u = *reinterpret_cast<const uint2*>(w);
  const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&u.x), b = *reinterpret_cast<const __nv_bfloat162*>(&u.y);
  return make_float4(__low2float(a), __high2float(a), __low2float(b), __high2float(b));
}
__device__ __forceinline__ void st4(float* y, float4 v) { *reinterpret_cast<float4*>(y) = v; }
__device__ __forceinline__ void st4(__nv_bfloat16* y, float4 v) {
  __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
  uint2 u; u.x = *reinterpret_cast<uint32_t*>(&a); u.y = *reinterpret_cast<uint32_t*>(&b);
  *reinterpret_cast<uint2*>(y) = u;
}
template <typename E, bool LN>
__global__ void __launch_bounds__(256) norm_f32in_vec_kernel(E* y, const float* x, const int32_t* rows, const E* w, int d, float eps, float offset, float out_scale) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float red[33];
  const int r = blockIdx.x, nvec = d >> 2;
  const float* src = x + (int64_t)(rows ? rows[r] : r) * d;
  float4 v[NV_MAX];
  float s = 0.f;
#pragma unroll
  for (int i = 0; i < NV_MAX; ++i) {
    const int c = threadIdx.x + i * 256;
    v[i] = c < nvec ? *reinterpret_cast<const float4*>(src + 4 * c) : make_float4(0.f, 0.f, 0.f, 0.f);
    if (LN) s += (v[i].x + v[i].y) + (v[i].z + v[i].w);
  }
  float mean = 0.f;
  if (LN) { mean = block_sum(s, red) / (float)d; __syncthreads(); }
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < NV_MAX; ++i) {
    if (threadIdx.x + i * 256 < nvec) {
      v[i].x -= mean; v[i].y -= mean; v[i].z -= mean; v[i].w -= mean;
      ss = fmaf(v[i].x, v[i].x, ss); ss = fmaf(v[i].y, v[i].y, ss); ss = fmaf(v[i].z, v[i].z, ss); ss = fmaf(v[i].w, v[i].w, ss);
    }
  }
  ss = block_sum(ss, red);
  const float inv = out_scale / sqrtf(ss / (float)d + eps);
#pragma unroll
  for (int i = 0; i < NV_MAX; ++i) {
    const int c = threadIdx.x + i * 256;
    if (c < nvec) {
      const float4 g = ldw4(w + 4 * c);
      st4(y + (int64_t)r * d + 4 * c, make_float4(v[i].x * inv * (offset + g.x), v[i].y * inv * (offset + g.y), v[i].z * inv * (offset + g.z), v[i].w * inv * (offset + g.w)));
    }
  }
}
template <bool LN>
static bool norm_vec(void* y, const float* x, const int32_t* rows, const void* w, int R, int d, float eps, float offset, float out_scale, int elt, cudaStream_t st,
                     cudaError_t* ce) {
  if (d % 4 || d > 4 * 256 * NV_MAX || (reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(y) & 15) || (reinterpret_cast<uintptr_t>(w) & 15)) return false;
  *ce = elt == KGE_ELT_F32
      ? launch_pdl(norm_f32in_vec_kernel<float, LN>, dim3(R), dim3(256), 0, st, (float*)y, x, rows, (const float*)w, d, eps, offset, out_scale)
      : launch_pdl(norm_f32in_vec_kernel<__nv_bfloat16, LN>, dim3(R), dim3(256), 0, st, (__nv_bfloat16*)y, x, rows, (const __nv_bfloat16*)w, d, eps, offset, out_scale);
  return true;
}

// weight-only layer norm of an fp32 row: mean first, then the mean of the squared deviations (no cancellation)
template <typename E>
__global__ void layernorm_f32in_kernel(E* y, const float* x, const int32_t* rows, const E* w, int d, float eps, float out_scale) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float red[33];
  const int r = blockIdx.x;
  const float* src = x + (int64_t)(rows ? rows[r] : r) * d;
  float s = 0.f;
  for (int c = threadIdx.x; c < d; c += blockDim.x) s += src[c];
  const float mean = block_sum(s, red) / (float)d;
  __syncthreads();
  float ss = 0.f;
  for (int c = threadIdx.x; c < d; c += blockDim.x) { const float v = src[c] - mean; ss = fmaf(v, v, ss); }
  ss = block_sum(ss, red);
  const float inv = out_scale / sqrtf(ss / (float)d + eps);
  for (int c = threadIdx.x; c < d; c += blockDim.x) stf(y + (int64_t)r * d + c, (src[c] - mean) * inv * ldf(w + c));
}
int layernorm_f32in(void* y, const float* x, const int32_t* rows, const void* w, int R, int d, float eps, float out_scale, int elt, cudaStream_t st) {
  if (R <= 0) return 0;
  cudaError_t ce;
  if (norm_vec<true>(y, x, rows, w, R, d, eps, 0.f, out_scale, elt, st, &ce)) { KGE_CUDA_OK(ce); return 0; }
  ce = elt == KGE_ELT_F32
      ? launch_pdl(layernorm_f32in_kernel<float>, dim3(R), dim3(256), 0, st, (float*)y, x, rows, (const float*)w, d, eps, out_scale)
      : launch_pdl(layernorm_f32in_kernel<__nv_bfloat16>, dim3(R), dim3(256), 0, st, (__nv_bfloat16*)y, x, rows, (const __nv_bfloat16*)w, d, eps, out_scale);
  KGE_CUDA_OK(ce);
  return 0;
}

template <typename E>
__global__ void residual_combine_kernel(float* res, CombineArgs a, int64_t n, int d) {
  pdl_launch_dependents();
  pdl_wait();
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t t = i / d; const int c = (int)(i % d);
    float s = 0.f;
    for (int k = 0; k < a.n; ++k) {
      const float f = a.rscale[k] ? a.scale[k] * a.rscale[k][t * a.rs_stride[k]] : a.scale[k];
      s = fmaf(f, ldf((const E*)a.src[k] + t * a.ld[k] + c), s);
    }
    res[i] += s;
  }
}
// four columns per thread: one float4 of the stream, one 8- or 16-byte piece of every source
template <typename E>
__global__ void residual_combine_vec_kernel(float* res, CombineArgs a, int64_t n4, int d4) {
  pdl_launch_dependents();
  pdl_wait();
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t t = i / d4; const int c = (int)(i % d4) * 4;
    float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int k = 0; k < a.n; ++k) {
      const float f = a.rscale[k] ? a.scale[k] * a.rscale[k][t * a.rs_stride[k]] : a.scale[k];
      const float4 v = ldw4((const E*)a.src[k] + t * a.ld[k] + c);
      s.x = fmaf(f, v.x, s.x); s.y = fmaf(f, v.y, s.y); s.z = fmaf(f, v.z, s.z); s.w = fmaf(f, v.w, s.w);
    }
    float4* dst = reinterpret_cast<float4*>(res) + i;
    float4 o = *dst;
    o.x += s.x; o.y += s.y; o.z += s.z; o.w += s.w;
    *dst = o;
  }
}
int residual_combine(float* res, const CombineArgs& a, int T, int d, int elt, cudaStream_t st) {
  if (T <= 0 || a.n <= 0) return 0;
  const int64_t n = (int64_t)T * d;
  bool vec = d % 4 == 0 && (reinterpret_cast<uintptr_t>(res) & 15) == 0;
  for (int k = 0; k < a.n; ++k) vec = vec && a.ld[k] % 4 == 0 && (reinterpret_cast<uintptr_t>(a.src[k]) & 15) == 0;
  if (vec) {
    const int grid4 = (int)std::min<int64_t>((n / 4 + 255) / 256, 148 * 16);
    cudaError_t ce4 = elt == KGE_ELT_F32 ? launch_pdl(residual_combine_vec_kernel<float>, dim3(grid4), dim3(256), 0, st, res, a, n / 4, d / 4)
                                         : launch_pdl(residual_combine_vec_kernel<__nv_bfloat16>, dim3(grid4), dim3(256), 0, st, res, a, n / 4, d / 4);
    KGE_CUDA_OK(ce4);
    return 0;
  }
  const int grid = (int)std::min<int64_t>((n + 255) / 256, 148 * 8);
  cudaError_t ce = elt == KGE_ELT_F32 ? launch_pdl(residual_combine_kernel<float>, dim3(grid), dim3(256), 0, st, res, a, n, d)
                                      : launch_pdl(residual_combine_kernel<__nv_bfloat16>, dim3(grid), dim3(256), 0, st, res, a, n, d);
  KGE_CUDA_OK(ce);
  return 0;
}

__global__ void logits_to_elt16_kernel(uint16_t* out, const float* in, int R, int V, int ld, bool f16) {
  pdl_launch_dependents();
  pdl_wait();
  const int64_t n = (int64_t)R * V;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = i / V; const int c = (int)(i % V);
    out[r * ld + c] = f16 ? __half_as_ushort(__float2half_rn(in[i])) : __bfloat16_as_ushort(__float2bfloat16_rn(in[i]));
  }
}
int logits_to_elt16(void* out, const float* in, int R, int V, int ld_out, bool f16, cudaStream_t st) {
  if (R <= 0) return 0;
  const int grid = (int)std::min<int64_t>(((int64_t)R * V + 255) / 256, 148 * 8);
  KGE_CUDA_OK(launch_pdl(logits_to_elt16_kernel, dim3(grid), dim3(256), 0, st, (uint16_t*)out, in, R, V, ld_out, f16));
  return 0;
}

__global__ void elt16_to_f32_kernel(float* out, const __nv_bfloat16* in, int64_t n) {
  pdl_launch_dependents();
  pdl_wait();
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) out[i] = __bfloat162float(in[i]);
}
int elt16_to_f32(float* out, const void* in_bf16, int64_t n, cudaStream_t st) {
  if (n <= 0) return 0;
  KGE_CUDA_OK(launch_pdl(elt16_to_f32_kernel, dim3((unsigned)std::min<int64_t>((n + 255) / 256, 148 * 8)), dim3(256), 0, st, out, (const __nv_bfloat16*)in_bf16, n));
  return 0;
}


__device__ __forceinline__ float softcap_f(float v, float cap) { return cap * tanhf(v / cap); }
__global__ void softcap_rows_kernel(float* l32, __nv_bfloat16* l16, int R, int V, int ld16, float cap) {
  pdl_launch_dependents();
  pdl_wait();
  const int64_t n = (int64_t)R * V;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = i / V; const int c = (int)(i % V);
    const float v = softcap_f(l16 ? __bfloat162float(l16[r * ld16 + c]) : l32[i], cap);
    if (l32) l32[i] = v;
    if (l16) l16[r * ld16 + c] = __float2bfloat16_rn(v);
  }
}
int softcap_rows(float* l32, void* l16, int R, int V, int ld16, float cap, cudaStream_t st) {
  if (R <= 0 || cap <= 0.f) return 0;
  const int grid = (int)std::min<int64_t>(((int64_t)R * V + 255) / 256, 148 * 8);
  KGE_CUDA_OK(launch_pdl(softcap_rows_kernel, dim3(grid), dim3(256), 0, st, l32, (__nv_bfloat16*)l16, R, V, ld16, cap));
  return 0;
}

}  // namespace kge
