// Paged attention with a linear distance bias per head, a chunk mask, an optional soft cap of the scores and an optional
// sink logit per head in the softmax denominator, for any key / value head size, in bfloat16 or float32 storage.  One warp per (query row, head): 32 keys at a time, one key per lane for the scores (q in shared
// memory), softmax statistics in fp32 across the warp, then the lanes split the value columns.  Only keys of the
// query's own chunk are read, so the cost per query is bounded by the chunk size whatever the context length.
#include "common.cuh"
#include "elt_access.cuh"
#include "hybrid_ops.h"

namespace kge {

constexpr int ATT_WARPS = 4, ATT_MAXV = 8;   // value columns per lane: vdim <= 32 * ATT_MAXV

// Keys of a row with a window: first the `prefix` keys - kept first tokens that have left the window (their own rows of
// the caches) or pooled blocks that lie wholly before it (rows of the pooled caches) - then the window's tokens.
__device__ __forceinline__ int prefix_keys(const AttnBiasArgs& a, int i) {
  if (a.window <= 0 || i < a.window) return 0;
  const int before = i - a.window + 1;              // positions 0 .. before - 1 have left the window
  return a.pool > 0 ? before / a.pool : min(a.keep_first, before);
}
__device__ __forceinline__ int window_lo(const AttnBiasArgs& a, int i) {
  const int lo = a.chunk > 0 ? (i / a.chunk) * a.chunk : 0;
  return a.window > 0 ? max(lo, i - a.window + 1) : lo;
}
// the cache row of prefix key u of a request (pooled caches when pool > 0)
__device__ __forceinline__ int64_t prefix_row(const AttnBiasArgs& a, const int32_t* bt, int g, int u) {
  if (a.pool > 0) return ((int64_t)bt[u / a.pool_slots] * a.G + g) * a.pool_slots + u % a.pool_slots;
  return ((int64_t)bt[u / a.block_size] * a.G + g) * a.block_size + u % a.block_size;
}

template <typename E>
__global__ void __launch_bounds__(ATT_WARPS * 32) attn_bias_chunk_kernel(AttnBiasArgs a) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ float qs_all[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t item = (int64_t)blockIdx.x * ATT_WARPS + warp;
  if (item >= (int64_t)a.T * a.H) return;
  const int t = (int)(item / a.H), h = (int)(item % a.H);
  float* qs = qs_all + warp * a.dim;
  const E* q = (const E*)a.q + (int64_t)t * a.ldq + h * a.dim;
  for (int d = lane; d < a.dim; d += 32) qs[d] = ldf(q + d);
  __syncwarp();
  const int b = a.token_req[t], i = a.positions[t];
  const int lo = window_lo(a, i), npre = prefix_keys(a, i);
  const int g = h / (a.H / a.G);
  const float slope = a.bias_span > 0.f ? exp2f(-a.bias_span * (float)(h + 1) / (float)a.H) : 0.f;
  const int32_t* bt = a.block_table + (int64_t)b * a.max_blocks;
  const E* kc = (const E*)a.k_cache;
  const E* vc = (const E*)a.v_cache;
  const bool pooled = a.pool > 0;
  const E* pkc = pooled ? (const E*)a.pk_cache : kc;
  const E* pvc = pooled ? (const E*)a.pv_cache : vc;
  float m = -INFINITY, l = 0.f, o[ATT_MAXV];
#pragma unroll
  for (int c = 0; c < ATT_MAXV; ++c) o[c] = 0.f;
  // the row's keys in one list: npre prefix keys, then positions lo .. i
  const int nkeys = npre + (i - lo + 1);
  for (int u0 = 0; u0 < nkeys; u0 += 32) {
    const int u = u0 + lane;
    const bool valid = u < nkeys, pre = u < npre;
    const int j = lo + (u - npre);
    int64_t row = 0;
    float s = -INFINITY;
    if (valid) {
      row = pre ? prefix_row(a, bt, g, u) : ((int64_t)bt[j / a.block_size] * a.G + g) * a.block_size + j % a.block_size;
      const E* kr = (pre ? pkc : kc) + row * a.dim;
      float acc = 0.f;
      for (int d = 0; d < a.dim; ++d) acc = fmaf(qs[d], ldf(kr + d), acc);
      acc *= a.scale;
      if (a.softcap > 0.f) acc = a.softcap * tanhf(acc / a.softcap);
      s = pre ? acc : acc - slope * (float)(i - j);
    }
    const float mn = fmaxf(m, warp_max(s));
    const float p = valid ? expf(s - mn) : 0.f;
    const float corr = expf(m - mn);            // m = -inf on the first tile: exp(-inf) = 0
    l = l * corr + warp_sum(p);
    m = mn;
#pragma unroll
    for (int c = 0; c < ATT_MAXV; ++c) o[c] *= corr;
    const int cnt = min(32, nkeys - u0);
    for (int jj = 0; jj < cnt; ++jj) {
      const float pj = __shfl_sync(0xffffffffu, p, jj);
      const int64_t rj = __shfl_sync(0xffffffffu, row, jj);
      const E* vr = (u0 + jj < npre ? pvc : vc) + rj * a.vdim;
#pragma unroll
      for (int c = 0; c < ATT_MAXV; ++c) {
        const int col = c * 32 + lane;
        if (col < a.vdim) o[c] = fmaf(pj, ldf(vr + col), o[c]);
      }
    }
  }
  if (a.sinks) {                                // the sink logit joins the denominator: no key, no value
    const float sk = a.sinks[h], mn = fmaxf(m, sk), corr = expf(m - mn);
    l = l * corr + expf(sk - mn);
#pragma unroll
    for (int c = 0; c < ATT_MAXV; ++c) o[c] *= corr;
  }
  const float inv = a.out_scale / l;
  E* out = (E*)a.out + (int64_t)t * a.ldo + h * a.vdim;
#pragma unroll
  for (int c = 0; c < ATT_MAXV; ++c) {
    const int col = c * 32 + lane;
    if (col < a.vdim) stf(out + col, o[c] * inv);
  }
}

// ---------------------------------------------------------------------------------------------------------------
// bfloat16, head sizes that are multiples of 16 (keys) / 8 (values) up to 128: the same attention on the tensor cores
// (mma.sync m16n8k16).  A CTA owns 16 rows - consecutive (token, query head of one key/value head) pairs of one
// request, so neighbouring tokens and the heads of a group share every key tile - and its four warps take the 32-key
// tiles of the rows' chunk in turn: K and V of a tile are staged in the warp's own shared memory with 16-byte loads,
// S = Q K^T and O += P V are mma instructions with fp32 accumulators, bias, mask and softmax statistics stay in fp32,
// and the four partial results (m, l, O) are merged through shared memory at the end.  Decoding a single token is the
// same kernel with hpg rows in use: its four warps split the chunk's keys.
constexpr int AM_WARPS = 4, AM_KT = 32, AM_MAXD = 128, AM_PAD = 8;

__device__ __forceinline__ void mma_16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// tanh(x) = 1 - 2 / (e^(2x) + 1): absolute error of a few 1e-7 over the whole range (saturates cleanly at +-1)
__device__ __forceinline__ float tanh_fast(float x) {
  return 1.f - __fdividef(2.f, exp2f(fminf(x * 2.8853900817779268f, 100.f)) + 1.f);
}
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
  __nv_bfloat162 p = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&p);
}
__device__ __forceinline__ uint32_t pack2raw(__nv_bfloat16 lo, __nv_bfloat16 hi) {
  return (uint32_t)__bfloat16_as_ushort(lo) | ((uint32_t)__bfloat16_as_ushort(hi) << 16);
}

// ROWS = false: a CTA owns 16 rows and its warps split the key tiles (decoding, short pieces).  ROWS = true: a CTA owns
// 64 rows, 16 per warp, and every key tile is staged once for all four warps (prompts).
template <bool ROWS>
__global__ void __launch_bounds__(AM_WARPS * 32) attn_bias_mma_kernel(AttnBiasArgs a, int req0) {
  pdl_launch_dependents();
  pdl_wait();
  typedef __nv_bfloat16 E;
  extern __shared__ __align__(16) unsigned char am_smem[];
  const int b = req0 + blockIdx.z, g = blockIdx.y, hpg = a.H / a.G;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, qr = lane >> 2, qc = (lane & 3) * 2;
  const int rs = a.qsl[b], nrows = (a.qsl[b + 1] - rs) * hpg, Rc = blockIdx.x * (ROWS ? 16 * AM_WARPS : 16);
  if (Rc >= nrows) return;
  const int R0 = ROWS ? Rc + warp * 16 : Rc;               // may lie beyond the request's rows: such a warp only helps staging
  const int dim = a.dim, vdim = a.vdim, ksteps = dim >> 4, vtiles = vdim >> 3;
  const int kst = dim + AM_PAD, vst = vdim + AM_PAD;                 // shared row strides (elements)
  const size_t region = (size_t)AM_KT * (kst + vst) * sizeof(E);
  E* Ks = reinterpret_cast<E*>(am_smem + (ROWS ? 0 : warp) * region);
  E* Vs = Ks + AM_KT * kst;
  // this thread's two rows: qr and qr + 8 of the tile
  int pos[2], lo[2], tok[2], head[2], npre[2];
  float slope2[2];
  const float log2e = 1.4426950408889634f;
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int r = R0 + qr + 8 * h;
    const bool valid = r < nrows;
    tok[h] = rs + (valid ? r : nrows - 1) / hpg;
    head[h] = g * hpg + (valid ? r : nrows - 1) % hpg;
    pos[h] = valid ? a.positions[tok[h]] : -1;                       // -1: no key is visible, the row is never written
    lo[h] = pos[h] >= 0 ? window_lo(a, pos[h]) : 0;
    npre[h] = pos[h] >= 0 ? prefix_keys(a, pos[h]) : 0;
    slope2[h] = a.bias_span > 0.f ? exp2f(-a.bias_span * (float)(head[h] + 1) / (float)a.H) * log2e : 0.f;
  }
  const int pos_first = a.positions[rs + Rc / hpg], pos_last = a.positions[rs + min(Rc + (ROWS ? 16 * AM_WARPS : 16) - 1, nrows - 1) / hpg];
  const int lo_min = window_lo(a, pos_first);
  // prefix keys (kept first tokens or pooled blocks) come first, in tiles of their own; the last row of the CTA sees the most
  const int pre_cta = prefix_keys(a, pos_last), ptiles = (pre_cta + AM_KT - 1) / AM_KT;
  const int ntiles = ptiles + (pos_last - lo_min + AM_KT) / AM_KT;
  // the keys this warp's own rows can see (ROWS: tiles outside are staged for the others but not computed here)
  // (the same for every lane of the warp: the mma instructions below need all 32 lanes on one path)
  const bool wany = R0 < nrows;
  const int own_hi = wany ? a.positions[rs + min(R0 + 15, nrows - 1) / hpg] : -1;
  const int own_first = wany ? a.positions[rs + R0 / hpg] : 0;
  const int own_lo = window_lo(a, own_first), own_pre = wany ? prefix_keys(a, own_hi) : 0;
  const float scale2 = a.scale * log2e;
  const float cap2 = a.softcap * log2e, cap_in = a.softcap > 0.f ? a.scale / a.softcap : 0.f;   // capped scores, in units of log 2
  uint32_t qf[AM_MAXD / 16][4];
#pragma unroll
  for (int ks = 0; ks < AM_MAXD / 16; ++ks) {
    if (ks < ksteps) {
      const E* q0 = (const E*)a.q + (int64_t)tok[0] * a.ldq + head[0] * dim + ks * 16 + qc;
      const E* q1 = (const E*)a.q + (int64_t)tok[1] * a.ldq + head[1] * dim + ks * 16 + qc;
      qf[ks][0] = pos[0] >= 0 ? *reinterpret_cast<const uint32_t*>(q0) : 0u;
      qf[ks][1] = pos[1] >= 0 ? *reinterpret_cast<const uint32_t*>(q1) : 0u;
      qf[ks][2] = pos[0] >= 0 ? *reinterpret_cast<const uint32_t*>(q0 + 8) : 0u;
      qf[ks][3] = pos[1] >= 0 ? *reinterpret_cast<const uint32_t*>(q1 + 8) : 0u;
    } else {
      qf[ks][0] = qf[ks][1] = qf[ks][2] = qf[ks][3] = 0u;
    }
  }
  float o[AM_MAXD / 8][4];
#pragma unroll
  for (int v = 0; v < AM_MAXD / 8; ++v) o[v][0] = o[v][1] = o[v][2] = o[v][3] = 0.f;
  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
  const int32_t* bt = a.block_table + (int64_t)b * a.max_blocks;
  const int kseg = dim >> 3, vseg = vdim >> 3;
  for (int kt = ROWS ? 0 : warp; kt < ntiles; kt += ROWS ? 1 : AM_WARPS) {
    const bool ptile = kt < ptiles;                         // a tile of prefix keys: j0 counts them from 0
    const int j0 = ptile ? kt * AM_KT : lo_min + (kt - ptiles) * AM_KT;
    const E* kc = (const E*)(ptile && a.pool > 0 ? a.pk_cache : a.k_cache);
    const E* vc = (const E*)(ptile && a.pool > 0 ? a.pv_cache : a.v_cache);
    if (ROWS) __syncthreads();                              // the previous tile has been read by every warp
    // stage the tile: lane i knows where key j0 + i lives; the 16-byte pieces of a row are fetched by consecutive lanes
    const int jl = j0 + lane;
    int64_t myrow = -1;
    if (ptile) { if (jl < pre_cta) myrow = prefix_row(a, bt, g, jl); }
    else if (jl <= pos_last) myrow = ((int64_t)bt[jl / a.block_size] * a.G + g) * a.block_size + jl % a.block_size;
    const int sid = ROWS ? threadIdx.x : lane, sstep = ROWS ? AM_WARPS * 32 : 32;
    // four 16-byte pieces (eight where one warp stages a whole tile: decoding) are requested before the first is stored, so
    // a tile costs a few memory round trips, not one per piece (whole warps run the loops: the shuffle needs every lane)
    constexpr int SU = ROWS ? 4 : 8;
    for (int idx0 = 0; idx0 < AM_KT * kseg; idx0 += SU * sstep) {
      uint4 v[SU]; int dst[SU];
#pragma unroll
      for (int u = 0; u < SU; ++u) {
        const int idx = min(idx0 + u * sstep + sid, AM_KT * kseg - 1);
        const int key = idx / kseg, seg = idx % kseg;
        const int64_t row = __shfl_sync(0xffffffffu, myrow, key);
        v[u] = make_uint4(0u, 0u, 0u, 0u);
        if (row >= 0) v[u] = *reinterpret_cast<const uint4*>(kc + row * dim + seg * 8);
        dst[u] = key * kst + seg * 8;
      }
#pragma unroll
      for (int u = 0; u < SU; ++u) *reinterpret_cast<uint4*>(Ks + dst[u]) = v[u];
    }
    for (int idx0 = 0; idx0 < AM_KT * vseg; idx0 += SU * sstep) {
      uint4 v[SU]; int dst[SU];
#pragma unroll
      for (int u = 0; u < SU; ++u) {
        const int idx = min(idx0 + u * sstep + sid, AM_KT * vseg - 1);
        const int key = idx / vseg, seg = idx % vseg;
        const int64_t row = __shfl_sync(0xffffffffu, myrow, key);
        v[u] = make_uint4(0u, 0u, 0u, 0u);
        if (row >= 0) v[u] = *reinterpret_cast<const uint4*>(vc + row * vdim + seg * 8);
        dst[u] = key * vst + seg * 8;
      }
#pragma unroll
      for (int u = 0; u < SU; ++u) *reinterpret_cast<uint4*>(Vs + dst[u]) = v[u];
    }
    if (ROWS) __syncthreads(); else __syncwarp();
    if (ROWS && (ptile ? j0 >= own_pre : (j0 > own_hi || j0 + AM_KT <= own_lo))) continue;
    float sacc[4][4];
#pragma unroll
    for (int nt = 0; nt < 4; ++nt) sacc[nt][0] = sacc[nt][1] = sacc[nt][2] = sacc[nt][3] = 0.f;
#pragma unroll
    for (int ks = 0; ks < AM_MAXD / 16; ++ks) {
      if (ks < ksteps) {
#pragma unroll
        for (int nt = 0; nt < 4; ++nt) {
          const E* kp = Ks + (nt * 8 + qr) * kst + ks * 16 + qc;
          mma_16816(sacc[nt], qf[ks], *reinterpret_cast<const uint32_t*>(kp), *reinterpret_cast<const uint32_t*>(kp + 8));
        }
      }
    }
    // bias, mask, running maximum (exponent base 2)
    float tmax[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int nt = 0; nt < 4; ++nt)
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const int h = c >> 1, j = j0 + nt * 8 + qc + (c & 1);
        const bool vis = ptile ? j < npre[h] : (j <= pos[h] && j >= lo[h]);
        float sc = sacc[nt][c] * scale2;
        if (cap2 > 0.f) sc = cap2 * tanh_fast(sacc[nt][c] * cap_in);
        const float sv = vis ? (ptile ? sc : sc - slope2[h] * (float)(pos[h] - j)) : -INFINITY;
        sacc[nt][c] = sv;
        tmax[h] = fmaxf(tmax[h], sv);
      }
    float corr[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      tmax[h] = fmaxf(tmax[h], __shfl_xor_sync(0xffffffffu, tmax[h], 1));
      tmax[h] = fmaxf(tmax[h], __shfl_xor_sync(0xffffffffu, tmax[h], 2));
      const float mn = fmaxf(m[h], tmax[h]);
      corr[h] = mn == -INFINITY ? 1.f : exp2f(m[h] - mn);
      m[h] = mn;
      l[h] *= corr[h];
    }
#pragma unroll
    for (int nt = 0; nt < 4; ++nt)
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const int h = c >> 1;
        const float p = sacc[nt][c] == -INFINITY ? 0.f : exp2f(sacc[nt][c] - m[h]);
        sacc[nt][c] = p;
        l[h] += p;
      }
#pragma unroll
    for (int v = 0; v < AM_MAXD / 8; ++v) { o[v][0] *= corr[0]; o[v][1] *= corr[0]; o[v][2] *= corr[1]; o[v][3] *= corr[1]; }
    uint32_t pf[2][4];
#pragma unroll
    for (int kk = 0; kk < 2; ++kk) {
      pf[kk][0] = pack2(sacc[2 * kk][0], sacc[2 * kk][1]);
      pf[kk][1] = pack2(sacc[2 * kk][2], sacc[2 * kk][3]);
      pf[kk][2] = pack2(sacc[2 * kk + 1][0], sacc[2 * kk + 1][1]);
      pf[kk][3] = pack2(sacc[2 * kk + 1][2], sacc[2 * kk + 1][3]);
    }
#pragma unroll
    for (int v = 0; v < AM_MAXD / 8; ++v) {
      if (v < vtiles) {
#pragma unroll
        for (int kk = 0; kk < 2; ++kk) {
          const E* vp = Vs + (kk * 16 + qc) * vst + v * 8 + qr;
          mma_16816(o[v], pf[kk], pack2raw(vp[0], vp[vst]), pack2raw(vp[8 * vst], vp[9 * vst]));
        }
      }
    }
    if (!ROWS) __syncwarp();
  }
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    l[h] += __shfl_xor_sync(0xffffffffu, l[h], 1);
    l[h] += __shfl_xor_sync(0xffffffffu, l[h], 2);
  }
  if (ROWS) {
    // each warp finished its own rows: normalise and store from the registers
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      if (pos[h] < 0) continue;
      float oc = 1.f;
      if (a.sinks) {
        const float sk = a.sinks[head[h]] * log2e, mn = fmaxf(m[h], sk);
        oc = exp2f(m[h] - mn);
        l[h] = l[h] * oc + exp2f(sk - mn);
      }
      const float inv = a.out_scale * oc / l[h];
      E* out = (E*)a.out + (int64_t)tok[h] * a.ldo + head[h] * vdim + qc;
#pragma unroll
      for (int v = 0; v < AM_MAXD / 8; ++v)
        if (v < vtiles) *reinterpret_cast<uint32_t*>(out + v * 8) = pack2(o[v][2 * h] * inv, o[v][2 * h + 1] * inv);
    }
    return;
  }
  // merge the four warps' partial results
  __syncthreads();                                          // every warp is done with its tiles: the regions are free
  float* Os = reinterpret_cast<float*>(am_smem + warp * region);      // [16][vdim]
  float* ML = reinterpret_cast<float*>(am_smem + AM_WARPS * region);  // [warps][2][16]
#pragma unroll
  for (int v = 0; v < AM_MAXD / 8; ++v) {
    if (v < vtiles) {
      Os[qr * vdim + v * 8 + qc] = o[v][0]; Os[qr * vdim + v * 8 + qc + 1] = o[v][1];
      Os[(qr + 8) * vdim + v * 8 + qc] = o[v][2]; Os[(qr + 8) * vdim + v * 8 + qc + 1] = o[v][3];
    }
  }
  if ((lane & 3) == 0) {
    ML[(warp * 2 + 0) * 16 + qr] = m[0]; ML[(warp * 2 + 0) * 16 + qr + 8] = m[1];
    ML[(warp * 2 + 1) * 16 + qr] = l[0]; ML[(warp * 2 + 1) * 16 + qr + 8] = l[1];
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < 16 * vdim; idx += AM_WARPS * 32) {
    const int r = idx / vdim, c = idx % vdim;
    if (R0 + r >= nrows) continue;
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < AM_WARPS; ++w) M = fmaxf(M, ML[(w * 2) * 16 + r]);
    const int row = R0 + r;
    float num = 0.f, den = 0.f;
    if (a.sinks) {
      const float sk = a.sinks[g * hpg + row % hpg] * log2e;
      M = fmaxf(M, sk);
      den = exp2f(sk - M);
    }
#pragma unroll
    for (int w = 0; w < AM_WARPS; ++w) {
      const float mw = ML[(w * 2) * 16 + r];
      const float f = mw == -INFINITY ? 0.f : exp2f(mw - M);
      num = fmaf(f, reinterpret_cast<const float*>(am_smem + w * region)[r * vdim + c], num);
      den = fmaf(f, ML[(w * 2 + 1) * 16 + r], den);
    }
    E* out = (E*)a.out + (int64_t)(rs + row / hpg) * a.ldo + (g * hpg + row % hpg) * vdim + c;
    *out = __float2bfloat16_rn(num / den * a.out_scale);
  }
}

int attn_bias_chunk(const AttnBiasArgs& a, cudaStream_t st) {
  if (a.T <= 0) return 0;
  KGE_REQUIRE(a.window >= 0 && (a.window > 0 || (a.keep_first == 0 && a.pool == 0)) && !(a.keep_first > 0 && a.pool > 0) && (a.window == 0 || a.bias_span == 0.f) &&
              (a.pool == 0 || (a.pk_cache && a.pv_cache && a.pool_slots > 0)),
              "attn_bias_chunk: window %d with %d kept tokens / pooled blocks of %d", a.window, a.keep_first, a.pool);
  if (a.elt == KGE_ELT_BF16 && a.max_q > 0 && a.dim % 16 == 0 && a.dim <= AM_MAXD && a.vdim % 8 == 0 && a.vdim <= AM_MAXD && a.ldq % 2 == 0 &&
      a.H % a.G == 0 && (reinterpret_cast<uintptr_t>(a.q) & 3) == 0 && a.B <= 65535 && a.G <= 65535) {
    const int hpg = a.H / a.G;
    const size_t smem = (size_t)AM_WARPS * AM_KT * (a.dim + a.vdim + 2 * AM_PAD) * 2 + (size_t)AM_WARPS * 2 * 16 * 4;
    static size_t smem_set = 0;                       // opt in once per size that needs more than the default 48 KB
    if (smem > 48 * 1024 && smem > smem_set) {
      KGE_CUDA_OK(cudaFuncSetAttribute(attn_bias_mma_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
      KGE_CUDA_OK(cudaFuncSetAttribute(attn_bias_mma_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
      smem_set = smem;
    }
    // the leading one-token requests, then the rest; 64-row CTAs where a request has that many rows and its output
    // pairs can be stored as 32-bit words
    const int D = std::min(std::max(a.num_decode, 0), a.B);
    if (D > 0) KGE_CUDA_OK(launch_pdl(attn_bias_mma_kernel<false>, dim3((hpg + 15) / 16, a.G, D), dim3(AM_WARPS * 32), smem, st, a, 0));
    if (D < a.B) {
      const int rows = a.max_q * hpg;
      const bool wide = rows > 32 && a.ldo % 2 == 0 && a.vdim % 2 == 0 && (reinterpret_cast<uintptr_t>(a.out) & 3) == 0;
      if (wide) KGE_CUDA_OK(launch_pdl(attn_bias_mma_kernel<true>, dim3((rows + 16 * AM_WARPS - 1) / (16 * AM_WARPS), a.G, a.B - D), dim3(AM_WARPS * 32), smem, st, a, D));
      else KGE_CUDA_OK(launch_pdl(attn_bias_mma_kernel<false>, dim3((rows + 15) / 16, a.G, a.B - D), dim3(AM_WARPS * 32), smem, st, a, D));
    }
    return 0;
  }
  KGE_REQUIRE(a.vdim <= 32 * ATT_MAXV, "attn_bias_chunk: value head size %d > %d", a.vdim, 32 * ATT_MAXV);
  KGE_REQUIRE(a.dim <= 1024 && a.H % a.G == 0, "attn_bias_chunk: bad head sizes");
  const int64_t items = (int64_t)a.T * a.H;
  const dim3 grid((unsigned)((items + ATT_WARPS - 1) / ATT_WARPS)), block(ATT_WARPS * 32);
  const size_t smem = (size_t)ATT_WARPS * a.dim * 4;
  cudaError_t ce = a.elt == KGE_ELT_F32 ? launch_pdl(attn_bias_chunk_kernel<float>, grid, block, smem, st, a)
                                        : launch_pdl(attn_bias_chunk_kernel<__nv_bfloat16>, grid, block, smem, st, a);
  KGE_CUDA_OK(ce);
  return 0;
}

template <typename E>
__global__ void kv_write_any_kernel(const E* k, int ldk, const E* v, int ldv, const int64_t* slots, E* kc, E* vc, int G, int dim, int vdim, int bs) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const int64_t slot = slots[t];
  if (slot < 0) return;
  const int64_t blk = slot / bs, off = slot % bs;
  for (int c = threadIdx.x; c < G * dim; c += blockDim.x) {
    const int g = c / dim, d = c % dim;
    kc[((blk * G + g) * bs + off) * dim + d] = k[(int64_t)t * ldk + c];
  }
  for (int c = threadIdx.x; c < G * vdim; c += blockDim.x) {
    const int g = c / vdim, d = c % vdim;
    vc[((blk * G + g) * bs + off) * vdim + d] = v[(int64_t)t * ldv + c];
  }
}

int kv_write_any(const void* k, int ldk, const void* v, int ldv, const int64_t* slots, void* k_cache, void* v_cache, int T, int G,
                 int dim, int vdim, int block_size, int elt, cudaStream_t st) {
  if (T <= 0) return 0;
  cudaError_t ce = elt == KGE_ELT_F32
      ? launch_pdl(kv_write_any_kernel<float>, dim3(T), dim3(128), 0, st, (const float*)k, ldk, (const float*)v, ldv, slots, (float*)k_cache, (float*)v_cache, G, dim, vdim, block_size)
      : launch_pdl(kv_write_any_kernel<__nv_bfloat16>, dim3(T), dim3(128), 0, st, (const __nv_bfloat16*)k, ldk, (const __nv_bfloat16*)v, ldv, slots,
                   (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache, G, dim, vdim, block_size);
  KGE_CUDA_OK(ce);
  return 0;
}

// One block per (token, key/value head); only a token that ends a block of `pool` positions has work: the block's keys
// and values are read back from the caches (so what is averaged is what the attention reads), sixteen rows requested at a
// time, summed in fp32 in ascending position and divided by the count.  One column per thread and pass.
template <typename E>
__global__ void __launch_bounds__(256) pool_kv_write_kernel(PoolKvArgs a) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x, g = blockIdx.y, pos = a.positions[t];
  if ((pos + 1) % a.pool != 0) return;
  const int pb = pos / a.pool, p0 = pb * a.pool;
  const int32_t* bt = a.block_table + (int64_t)a.token_req[t] * a.max_blocks;
  const int64_t drow = ((int64_t)bt[pb / a.pool_slots] * a.G + g) * a.pool_slots + pb % a.pool_slots;
  for (int c = threadIdx.x; c < a.dim + a.vdim; c += blockDim.x) {
    const bool isk = c < a.dim;
    const int w = isk ? a.dim : a.vdim, dd = isk ? c : c - a.dim;
    const E* src = (const E*)(isk ? a.k_cache : a.v_cache);
    float acc = 0.f;
    for (int j0 = p0; j0 <= pos; j0 += 16) {
      float v[16];
#pragma unroll
      for (int u = 0; u < 16; ++u) {
        const int j = j0 + u;
        v[u] = j <= pos ? ldf(src + (((int64_t)bt[j / a.block_size] * a.G + g) * a.block_size + j % a.block_size) * w + dd) : 0.f;
      }
#pragma unroll
      for (int u = 0; u < 16; ++u) acc += v[u];
    }
    E* dst = (E*)(isk ? a.pk_cache : a.pv_cache);
    stf(dst + drow * w + dd, acc / (float)a.pool);
  }
}

int pool_kv_write(const PoolKvArgs& a, cudaStream_t st) {
  if (a.T <= 0) return 0;
  KGE_REQUIRE(a.pool >= 1 && a.pool_slots >= 1 && a.pool_slots * a.pool >= a.block_size && a.G <= 65535, "pool_kv_write: blocks of %d positions, %d entries per page of %d", a.pool, a.pool_slots, a.block_size);
  cudaError_t ce = a.elt == KGE_ELT_F32 ? launch_pdl(pool_kv_write_kernel<float>, dim3(a.T, a.G), dim3(256), 0, st, a)
                                        : launch_pdl(pool_kv_write_kernel<__nv_bfloat16>, dim3(a.T, a.G), dim3(256), 0, st, a);
  KGE_CUDA_OK(ce);
  return 0;
}

}  // namespace kge
