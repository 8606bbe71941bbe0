// Mixture-of-experts routing: fp32 router logits (optional bias), sigmoid or softmax scores or the raw logits with a
// softmax over the chosen ones, top-k choice, and the grouping of
// (token, choice) pairs by expert that the grouped linear layer consumes.  Which rows an expert gets is all that the
// grouping decides: a pair's result does not depend on its place in the group, and the pairs of a token are summed in
// choice order afterwards, so the routing order never shows in the output.
#include "common.cuh"
#include "elt_access.cuh"
#include "hybrid_ops.h"

namespace kge {

// One lane's share of the dot product of two rows, 16 bytes per load where the rows allow (the same order of summation
// for a row whatever the launch holds)
__device__ __forceinline__ float dot_part(const __nv_bfloat16* h, const __nv_bfloat16* w, int d, int lane, bool vec) {
  float acc = 0.f;
  if (vec) {
    for (int k = lane * 8; k < d; k += 256) {
      const uint4 a = *reinterpret_cast<const uint4*>(h + k), b = *reinterpret_cast<const uint4*>(w + k);
      const __nv_bfloat162* a2 = reinterpret_cast<const __nv_bfloat162*>(&a);
      const __nv_bfloat162* b2 = reinterpret_cast<const __nv_bfloat162*>(&b);
#pragma unroll
      for (int j = 0; j < 4; ++j) { const float2 x = __bfloat1622float2(a2[j]), y = __bfloat1622float2(b2[j]); acc = fmaf(x.x, y.x, acc); acc = fmaf(x.y, y.y, acc); }
    }
  } else {
    for (int k = lane; k < d; k += 32) acc = fmaf(__bfloat162float(h[k]), __bfloat162float(w[k]), acc);
  }
  return acc;
}
__device__ __forceinline__ float dot_part(const float* h, const float* w, int d, int lane, bool vec) {
  float acc = 0.f;
  if (vec) {
    for (int k = lane * 4; k < d; k += 128) {
      const float4 a = *reinterpret_cast<const float4*>(h + k), b = *reinterpret_cast<const float4*>(w + k);
      acc = fmaf(a.x, b.x, acc); acc = fmaf(a.y, b.y, acc); acc = fmaf(a.z, b.z, acc); acc = fmaf(a.w, b.w, acc);
    }
  } else {
    for (int k = lane; k < d; k += 32) acc = fmaf(h[k], w[k], acc);
  }
  return acc;
}

// One block per token: its eight warps share the experts' dot products (fp32, lanes summed by shuffles - the same order
// whatever the launch holds) and, where asked, one more row whose sigmoid is a per-token gate; then the first warp picks
// the top-k, each lane scanning its share of the scores.
template <typename E>
__global__ void __launch_bounds__(256) moe_score_kernel(MoeRouteArgs a) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ float sc[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, t = blockIdx.x;
  const E* h = (const E*)a.h + (int64_t)t * a.ldh;
  constexpr int per = 16 / (int)sizeof(E);
  const bool vec = a.d % per == 0 && a.ldh % per == 0 && (reinterpret_cast<uintptr_t>(a.h) & 15) == 0 && (reinterpret_cast<uintptr_t>(a.w_router) & 15) == 0 &&
                   (reinterpret_cast<uintptr_t>(a.w_extra) & 15) == 0;
  const int nrows = a.E + (a.w_extra ? 1 : 0);
  for (int e = warp; e < nrows; e += 8) {
    const E* w = e < a.E ? (const E*)a.w_router + (int64_t)e * a.d : (const E*)a.w_extra;
    const float acc = warp_sum(dot_part(h, w, a.d, lane, vec));
    if (lane == 0) {
      if (e < a.E) sc[e] = a.b_router ? acc + ldf((const E*)a.b_router + e) : acc;
      else a.extra_sigmoid[t] = 1.f / (1.f + expf(-acc));
    }
  }
  __syncthreads();
  if (warp != 0) return;
  if (a.score_fn == 0) {
    for (int e = lane; e < a.E; e += 32) sc[e] = 1.f / (1.f + expf(-sc[e]));
  } else if (a.score_fn == 1) {
    float mx = -INFINITY;
    for (int e = lane; e < a.E; e += 32) mx = fmaxf(mx, sc[e]);
    mx = warp_max(mx);
    float sum = 0.f;
    for (int e = lane; e < a.E; e += 32) { const float p = expf(sc[e] - mx); sc[e] = p; sum += p; }
    sum = warp_sum(sum);
    __syncwarp();
    for (int e = lane; e < a.E; e += 32) sc[e] /= sum;
  }
  __syncwarp();
  int32_t* ce = a.choice_expert + (int64_t)t * a.top;
  float* cw = a.choice_weight + (int64_t)t * a.top;
  for (int k = 0; k < a.top; ++k) {
    // the largest score not yet taken, the lower index on a tie; a taken score is marked -inf in shared memory
    float bv = -INFINITY; int best = 0x7fffffff;
    for (int e = lane; e < a.E; e += 32) { const float v = sc[e]; if (v > bv) { bv = v; best = e; } }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, off);
      const int oi = __shfl_xor_sync(0xffffffffu, best, off);
      if (ov > bv || (ov == bv && oi < best)) { bv = ov; best = oi; }
    }
    if (lane == 0) {
      if (best == 0x7fffffff) {      // scores that are not numbers (or all taken): the lowest index not chosen yet, weight 0
        best = 0;
        for (bool again = true; again;) { again = false; for (int q = 0; q < k; ++q) if (ce[q] == best) { ++best; again = true; } }
        bv = 0.f;
      }
      ce[k] = best; cw[k] = bv;
      sc[best] = -INFINITY;
    }
    __syncwarp();
  }
  if (lane == 0) {
    if (a.score_fn == 2) {          // softmax over the chosen logits only (the first choice holds the largest)
      const float mx = cw[0];
      float total = 0.f;
      for (int k = 0; k < a.top; ++k) { const float p = expf(cw[k] - mx); cw[k] = p; total += p; }
      for (int k = 0; k < a.top; ++k) cw[k] /= total;
    } else if (a.renorm) {
      float total = 0.f;
      for (int k = 0; k < a.top; ++k) total += cw[k];
      for (int k = 0; k < a.top; ++k) cw[k] /= total;
    }
    if (a.weight_scale != 1.f) for (int k = 0; k < a.top; ++k) cw[k] *= a.weight_scale;
  }
}

__global__ void __launch_bounds__(1024) moe_group_kernel(MoeRouteArgs a) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ int cnt[];            // [E] counts, then [E] cursors
  int* cur = cnt + a.E;
  const int n = a.T * a.top;
  for (int e = threadIdx.x; e < a.E; e += blockDim.x) cnt[e] = 0;
  __syncthreads();
  for (int i = threadIdx.x; i < n; i += blockDim.x) atomicAdd(&cnt[a.choice_expert[i]], 1);
  __syncthreads();
  if (threadIdx.x == 0) {
    int off = 0;
    for (int e = 0; e < a.E; ++e) {
      a.group_off[e] = off; cur[e] = off;
      off += a.pad > 1 ? (cnt[e] + a.pad - 1) / a.pad * a.pad : cnt[e];
    }
    a.group_off[a.E] = off;
  }
  __syncthreads();
  if (a.pad > 1) {
    // padded groups: rows that carry no pair are marked (the gather writes zeros there, the scatter skips them), and every
    // tile of `pad` rows learns its expert; tiles beyond the last group compute on zero rows with the first expert's weights
    for (int i = threadIdx.x; i < a.rows_padded; i += blockDim.x) { a.perm_token[i] = -1; a.perm_dest[i] = -1; a.perm_weight[i] = 0.f; }
    for (int i = threadIdx.x; i < a.rows_padded / a.pad; i += blockDim.x) {
      int e = 0;
      while (e + 1 < a.E && i * a.pad >= a.group_off[e + 1]) ++e;
      a.tile_group[i] = i * a.pad < a.group_off[a.E] ? e : 0;
    }
    __syncthreads();
  }
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const int p = atomicAdd(&cur[a.choice_expert[i]], 1);
    a.perm_token[p] = i / a.top;
    a.perm_weight[p] = a.choice_weight[i];
    a.perm_dest[p] = i;
  }
}

__global__ void moe_gather_rows_kernel(__nv_bfloat16* xperm, const __nv_bfloat16* h, int ldh, const int32_t* tok, const float* w, int d) {
  pdl_launch_dependents();
  pdl_wait();
  const int p = blockIdx.x;
  if (tok[p] < 0) {                              // a padding row of a group
    for (int c = threadIdx.x; c < d; c += blockDim.x) xperm[(int64_t)p * d + c] = __float2bfloat16_rn(0.f);
    return;
  }
  const __nv_bfloat16* src = h + (int64_t)tok[p] * ldh;
  if (!w && d % 8 == 0 && ldh % 8 == 0) {        // plain copy of the row, 16 bytes at a time
    for (int c = threadIdx.x; c < d / 8; c += blockDim.x) reinterpret_cast<uint4*>(xperm + (int64_t)p * d)[c] = reinterpret_cast<const uint4*>(src)[c];
    return;
  }
  const float s = w ? w[p] : 1.f;
  for (int c = threadIdx.x; c < d; c += blockDim.x) xperm[(int64_t)p * d + c] = __float2bfloat16_rn(s * __bfloat162float(src[c]));
}
__global__ void moe_scatter_rows_kernel(__nv_bfloat16* out, const __nv_bfloat16* operm, const int32_t* dest, int d) {
  pdl_launch_dependents();
  pdl_wait();
  const int p = blockIdx.x;
  if (dest[p] < 0) return;
  if (d % 8 == 0) {
    for (int c = threadIdx.x; c < d / 8; c += blockDim.x) reinterpret_cast<uint4*>(out + (int64_t)dest[p] * d)[c] = reinterpret_cast<const uint4*>(operm + (int64_t)p * d)[c];
    return;
  }
  for (int c = threadIdx.x; c < d; c += blockDim.x) out[(int64_t)dest[p] * d + c] = operm[(int64_t)p * d + c];
}
int moe_gather_rows(void* xperm, const void* h, int ldh, const int32_t* perm_token, const float* perm_weight, int np, int d, cudaStream_t st) {
  if (np <= 0) return 0;
  KGE_CUDA_OK(launch_pdl(moe_gather_rows_kernel, dim3(np), dim3(256), 0, st, (__nv_bfloat16*)xperm, (const __nv_bfloat16*)h, ldh, perm_token, perm_weight, d));
  return 0;
}
int moe_scatter_rows(void* out, const void* operm, const int32_t* perm_dest, int np, int d, cudaStream_t st) {
  if (np <= 0) return 0;
  KGE_CUDA_OK(launch_pdl(moe_scatter_rows_kernel, dim3(np), dim3(256), 0, st, (__nv_bfloat16*)out, (const __nv_bfloat16*)operm, perm_dest, d));
  return 0;
}

int moe_route(const MoeRouteArgs& a, cudaStream_t st) {
  if (a.T <= 0) return 0;
  KGE_REQUIRE(a.E > 0 && a.top > 0 && a.top <= a.E && a.E <= 4096, "moe_route: %d experts, top %d", a.E, a.top);
  KGE_REQUIRE(a.pad <= 1 || (a.tile_group && a.rows_padded % a.pad == 0 && a.rows_padded >= a.T * a.top + a.E * (a.pad - 1)),
              "moe_route: padded groups need tile_group and %d rows or more", a.T * a.top + a.E * (a.pad - 1));
  cudaError_t ce = a.elt == KGE_ELT_F32 ? launch_pdl(moe_score_kernel<float>, dim3(a.T), dim3(256), (size_t)a.E * 4, st, a)
                                        : launch_pdl(moe_score_kernel<__nv_bfloat16>, dim3(a.T), dim3(256), (size_t)a.E * 4, st, a);
  KGE_CUDA_OK(ce);
  KGE_CUDA_OK(launch_pdl(moe_group_kernel, dim3(1), dim3(1024), (size_t)2 * a.E * 4, st, a));
  return 0;
}

}  // namespace kge
