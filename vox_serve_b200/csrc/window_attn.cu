// Softmax attention with a sliding window over a paged cache whose key and value heads may have different sizes,
// grouped query heads, rotary positions on a leading slice of every head in (even, odd) pairs, cross-layer value mixing
// and a sigmoid output gate.  Operands bf16 or fp32; scores, softmax and the output accumulation in fp32.
//
//   vb_rotary_table      cos / sin of position * frequency, evaluated in double and rounded once (the table is shared by
//                        every layer of a step that has the same rotary constants)
//   vb_qkv_rotary_append the tail of a fused q|k|v|gate projection: rotate q and k, mix v with the first mixing layer's
//                        values of the same token, write q, append k and the mixed v to the layer's pages
//   vb_window_attn       decode rows (and steps that mix them with prompt portions): a CTA per (token row, key/value
//                        head) whose K / V tiles serve all query heads of the group; for head groups or value sizes
//                        beyond its registers, one warp per (token row, query head).  Online softmax, gate, store.
//   vb_window_attn_tiled prompt portions: one CTA per (64 query rows of one request, query head), K/V tiles staged in
//                        shared memory and reused by all rows of the tile.
// Cache layout per layer: K [pages][page_size][kv_heads][dim], V [pages][page_size][kv_heads][vdim].
#include "../../include/vb_api.h"
#define VB_PDL_FAMILY 1
#include "common.cuh"

namespace vb {

template <typename T> __device__ __forceinline__ float wa_to_f(T v);
template <> __device__ __forceinline__ float wa_to_f<float>(float v) { return v; }
template <> __device__ __forceinline__ float wa_to_f<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T wa_from_f(float v);
template <> __device__ __forceinline__ float wa_from_f<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 wa_from_f<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

__global__ void rotary_table_kernel(float* __restrict__ cs, const int32_t* __restrict__ pos, const double* __restrict__ freq,
                                    int T, int half) {
  pdl_sync();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= T * half) return;
  const int t = i / half, j = i - t * half;
  double s, c;
  sincos(static_cast<double>(pos[t]) * freq[j], &s, &c);
  cs[(static_cast<size_t>(t) * 2) * half + j] = static_cast<float>(c);
  cs[(static_cast<size_t>(t) * 2 + 1) * half + j] = static_cast<float>(s);
}

struct QkvTailParams {
  const float* proj;      // [T][ldp]: q | k | v | (gate) columns
  int ldp, q_off, k_off, v_off;
  const float* cs;        // [T][2][half] or nullptr (no rotation)
  int half;               // rotated dims / 2
  void* q_out;            // [T][H * dim]
  void* k_cache;
  void* v_cache;
  const int32_t* row_req;
  const int32_t* pos;
  const int32_t* page_indptr;
  const int32_t* page_indices;
  int page_size, H, G, dim, vdim;
  int vmix;               // 0 none, 1 record v as the first mixing layer's values, 2 mix with them
  float* v_first;         // [T][G * vdim] fp32
  const float* lambda;    // device scalar
};

template <typename CT>
__global__ void qkv_rotary_append_kernel(QkvTailParams p) {
  pdl_sync();
  const int t = blockIdx.x;
  const float* row = p.proj + static_cast<size_t>(t) * p.ldp;
  const int b = p.row_req[t], ps = p.pos[t];
  const int page = p.page_indices[p.page_indptr[b] + ps / p.page_size];
  const size_t tok = static_cast<size_t>(page) * p.page_size + ps % p.page_size;
  const float* cs = p.cs ? p.cs + static_cast<size_t>(t) * 2 * p.half : nullptr;
  CT* q_out = static_cast<CT*>(p.q_out) + static_cast<size_t>(t) * p.H * p.dim;
  CT* k_out = static_cast<CT*>(p.k_cache) + tok * p.G * p.dim;
  CT* v_out = static_cast<CT*>(p.v_cache) + tok * p.G * p.vdim;
  // q and k: pairs (2i, 2i + 1) of the first 2 * half dims of every head are rotated, the rest pass
  const int pairs_per_head = (p.dim + 1) / 2;
  const int nq = p.H * pairs_per_head, nk = p.G * pairs_per_head;
  for (int i = threadIdx.x; i < nq + nk; i += blockDim.x) {
    const bool is_q = i < nq;
    const int j = is_q ? i : i - nq;
    const int h = j / pairs_per_head, pr = j - h * pairs_per_head;
    const float* src = row + (is_q ? p.q_off : p.k_off) + h * p.dim + 2 * pr;
    CT* dst = (is_q ? q_out : k_out) + h * p.dim + 2 * pr;
    const bool has2 = 2 * pr + 1 < p.dim;
    float u = src[0], v = has2 ? src[1] : 0.f;
    if (cs && pr < p.half) {
      const float c = cs[pr], s = cs[p.half + pr];
      const float nu = u * c - v * s, nv = v * c + u * s;
      u = nu;
      v = nv;
    }
    dst[0] = wa_from_f<CT>(u);
    if (has2) dst[1] = wa_from_f<CT>(v);
  }
  const int nv = p.G * p.vdim;
  float lam = 0.f;
  if (p.vmix == 2) lam = *p.lambda;
  for (int i = threadIdx.x; i < nv; i += blockDim.x) {
    float v = row[p.v_off + i];
    if (p.vmix == 1) p.v_first[static_cast<size_t>(t) * nv + i] = v;
    else if (p.vmix == 2) v = (1.f - lam) * v + lam * p.v_first[static_cast<size_t>(t) * nv + i];
    v_out[i] = wa_from_f<CT>(v);
  }
}

struct WindowAttnParams {
  const void* q;          // [T][H][dim]
  const void* k_cache;
  const void* v_cache;
  void* out;              // [T][H * vdim]
  const float* gate;      // [T][ld_gate] (+ column offset applied by the host) or nullptr
  int ld_gate;
  const int32_t* row_req;
  const int32_t* pos;
  const int32_t* page_indptr;
  const int32_t* page_indices;
  const int32_t* qo_indptr;   // tiled kernel: rows of request b are qo[b]..qo[b+1]
  const int32_t* tile_req;    // tiled kernel: request of tile i
  const int32_t* tile_row0;   // tiled kernel: first row of tile i
  int T, H, G, dim, vdim, page_size, window;   // window <= 0: every earlier position is visible
  float scale;
};

template <typename CT>
__device__ __forceinline__ float dot_row(const float* __restrict__ q, const CT* __restrict__ k, int dim);
template <>
__device__ __forceinline__ float dot_row<float>(const float* __restrict__ q, const float* __restrict__ k, int dim) {
  float s = 0.f;
  if ((dim & 3) == 0) {
    for (int d = 0; d < dim; d += 4) {
      const float4 kv = *reinterpret_cast<const float4*>(k + d);
      s = fmaf(q[d], kv.x, s); s = fmaf(q[d + 1], kv.y, s); s = fmaf(q[d + 2], kv.z, s); s = fmaf(q[d + 3], kv.w, s);
    }
  } else {
    for (int d = 0; d < dim; ++d) s = fmaf(q[d], k[d], s);
  }
  return s;
}
template <>
__device__ __forceinline__ float dot_row<__nv_bfloat16>(const float* __restrict__ q, const __nv_bfloat16* __restrict__ k,
                                                        int dim) {
  float s = 0.f;
  if ((dim & 7) == 0) {
    for (int d = 0; d < dim; d += 8) {
      const uint4 kv = *reinterpret_cast<const uint4*>(k + d);
      s = fmaf(q[d], bf16_lo(kv.x), s); s = fmaf(q[d + 1], bf16_hi(kv.x), s);
      s = fmaf(q[d + 2], bf16_lo(kv.y), s); s = fmaf(q[d + 3], bf16_hi(kv.y), s);
      s = fmaf(q[d + 4], bf16_lo(kv.z), s); s = fmaf(q[d + 5], bf16_hi(kv.z), s);
      s = fmaf(q[d + 6], bf16_lo(kv.w), s); s = fmaf(q[d + 7], bf16_hi(kv.w), s);
    }
  } else {
    for (int d = 0; d < dim; ++d) s = fmaf(q[d], __bfloat162float(k[d]), s);
  }
  return s;
}

constexpr int WA_WARPS = 4, WA_MAXU = 8;      // value heads up to 32 * WA_MAXU wide

template <typename CT>
__global__ void __launch_bounds__(WA_WARPS * 32) window_attn_kernel(WindowAttnParams p) {
  extern __shared__ float smf[];
  pdl_sync();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x * WA_WARPS + warp, h = blockIdx.y;
  if (t >= p.T) return;
  float* qs = smf + warp * p.dim;
  const CT* q = static_cast<const CT*>(p.q) + (static_cast<size_t>(t) * p.H + h) * p.dim;
  for (int d = lane; d < p.dim; d += 32) qs[d] = wa_to_f(q[d]) * p.scale;
  __syncwarp();
  const int b = p.row_req[t], ps = p.pos[t], g = h / (p.H / p.G);
  const int32_t* pages = p.page_indices + p.page_indptr[b];
  const int lo = p.window > 0 ? max(0, ps - p.window + 1) : 0;
  const CT* kc = static_cast<const CT*>(p.k_cache);
  const CT* vc = static_cast<const CT*>(p.v_cache);
  float m = -INFINITY, l = 0.f, acc[WA_MAXU];
#pragma unroll
  for (int u = 0; u < WA_MAXU; ++u) acc[u] = 0.f;
  for (int c = lo; c <= ps; c += 32) {
    const int kj = c + lane;
    const bool ok = kj <= ps;
    int tok = 0;
    float s = -INFINITY;
    if (ok) {
      tok = pages[kj / p.page_size] * p.page_size + kj % p.page_size;
      s = dot_row<CT>(qs, kc + (static_cast<size_t>(tok) * p.G + g) * p.dim, p.dim);
    }
    const float m_new = fmaxf(m, warp_max(s));
    const float corr = expf(m - m_new);          // m = -inf on the first chunk: exp(-inf) = 0
    const float pj = ok ? expf(s - m_new) : 0.f;
    l = l * corr + warp_sum(pj);
    m = m_new;
#pragma unroll
    for (int u = 0; u < WA_MAXU; ++u) acc[u] *= corr;
    const int n = min(32, ps - c + 1);
    for (int jj = 0; jj < n; ++jj) {
      const float pv = __shfl_sync(0xffffffffu, pj, jj);
      const int tk = __shfl_sync(0xffffffffu, tok, jj);
      const CT* vr = vc + (static_cast<size_t>(tk) * p.G + g) * p.vdim;
#pragma unroll
      for (int u = 0; u < WA_MAXU; ++u) {
        const int d = lane + 32 * u;
        if (d < p.vdim) acc[u] = fmaf(pv, wa_to_f(vr[d]), acc[u]);
      }
    }
  }
  const float inv = 1.f / l;
  CT* out = static_cast<CT*>(p.out) + static_cast<size_t>(t) * p.H * p.vdim + h * p.vdim;
  const float* gate = p.gate ? p.gate + static_cast<size_t>(t) * p.ld_gate + h * p.vdim : nullptr;
#pragma unroll
  for (int u = 0; u < WA_MAXU; ++u) {
    const int d = lane + 32 * u;
    if (d < p.vdim) {
      float o = acc[u] * inv;
      if (gate) o *= 1.f / (1.f + expf(-gate[d]));
      out[d] = wa_from_f<CT>(o);
    }
  }
}

// ------------------------------------------------------------------------------------------------------------------
// Prompt portions: CTA = (tile of up to 64 consecutive rows of ONE request, query head), 256 threads.  Key / value
// tiles of 32 positions are staged in shared memory as fp32 and shared by all rows; thread (r = tid / 4, c = tid % 4)
// owns row r and, in the score phase, keys c, c + 4, ...; in the output phase the value dims c, c + 4, ....
// The four threads of a row exchange through shuffles (they are neighbours in a warp).
// ------------------------------------------------------------------------------------------------------------------
constexpr int WT_ROWS = 64, WT_KEYS = 32, WT_MAXD = 64;   // per-thread value dims: vdim / 4 <= WT_MAXD

template <typename CT>
__global__ void __launch_bounds__(256) window_attn_tiled_kernel(WindowAttnParams p) {
  extern __shared__ float smf[];
  pdl_sync();
  const int b = p.tile_req[blockIdx.x], row0 = p.tile_row0[blockIdx.x], h = blockIdx.y;
  const int row_end = min(row0 + WT_ROWS, p.qo_indptr[b + 1]);
  const int nrows = row_end - row0;
  const int dk = p.dim, dv = p.vdim, dkp = dk + 1, dvp = dv + 1;
  float* Qs = smf;                               // [64][dk + 1]
  float* Ks = Qs + WT_ROWS * dkp;                // [32][dk + 1]
  float* Vs = Ks + WT_KEYS * dkp;                // [32][dv + 1]
  float* Ps = Vs + WT_KEYS * dvp;                // [64][33]
  const int tid = threadIdx.x, r = tid >> 2, c = tid & 3;
  const int g = h / (p.H / p.G);
  const CT* q = static_cast<const CT*>(p.q);
  for (int i = tid; i < WT_ROWS * dk; i += 256) {
    const int rr = i / dk, d = i - rr * dk;
    Qs[rr * dkp + d] = rr < nrows ? wa_to_f(q[(static_cast<size_t>(row0 + rr) * p.H + h) * dk + d]) * p.scale : 0.f;
  }
  const int pos0 = p.pos[row0], pos_last = pos0 + nrows - 1;     // rows of a portion are consecutive positions
  const int my_pos = pos0 + r;
  const bool row_ok = r < nrows;
  const int my_lo = p.window > 0 ? max(0, my_pos - p.window + 1) : 0;
  const int lo = p.window > 0 ? max(0, pos0 - p.window + 1) : 0;
  const int32_t* pages = p.page_indices + p.page_indptr[b];
  const CT* kc = static_cast<const CT*>(p.k_cache);
  const CT* vc = static_cast<const CT*>(p.v_cache);
  float m = -INFINITY, l = 0.f;
  float acc[WT_MAXD];
#pragma unroll
  for (int u = 0; u < WT_MAXD; ++u) acc[u] = 0.f;
  const int nd = (dv + 3) / 4;
  for (int c0 = lo; c0 <= pos_last; c0 += WT_KEYS) {
    __syncthreads();
    for (int i = tid; i < WT_KEYS * dk; i += 256) {
      const int kk = i / dk, d = i - kk * dk, kj = c0 + kk;
      float v = 0.f;
      if (kj <= pos_last) {
        const size_t tok = static_cast<size_t>(pages[kj / p.page_size]) * p.page_size + kj % p.page_size;
        v = wa_to_f(kc[(tok * p.G + g) * dk + d]);
      }
      Ks[kk * dkp + d] = v;
    }
    for (int i = tid; i < WT_KEYS * dv; i += 256) {
      const int kk = i / dv, d = i - kk * dv, kj = c0 + kk;
      float v = 0.f;
      if (kj <= pos_last) {
        const size_t tok = static_cast<size_t>(pages[kj / p.page_size]) * p.page_size + kj % p.page_size;
        v = wa_to_f(vc[(tok * p.G + g) * dv + d]);
      }
      Vs[kk * dvp + d] = v;
    }
    __syncthreads();
    // scores of this thread's 8 keys
    float s[WT_KEYS / 4];
    float mx = -INFINITY;
#pragma unroll
    for (int e = 0; e < WT_KEYS / 4; ++e) {
      const int kk = c + 4 * e, kj = c0 + kk;
      float a = 0.f;
      const float* qr = Qs + r * dkp;
      const float* kr = Ks + kk * dkp;
      for (int d = 0; d < dk; ++d) a = fmaf(qr[d], kr[d], a);
      const bool vis = row_ok && kj <= my_pos && kj >= my_lo;
      s[e] = vis ? a : -INFINITY;
      mx = fmaxf(mx, s[e]);
    }
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
    const float m_new = fmaxf(m, mx);
    const float corr = m_new == -INFINITY ? 1.f : expf(m - m_new);
    float sum = 0.f;
#pragma unroll
    for (int e = 0; e < WT_KEYS / 4; ++e) {
      const float pj = s[e] == -INFINITY ? 0.f : expf(s[e] - m_new);
      Ps[r * (WT_KEYS + 1) + c + 4 * e] = pj;
      sum += pj;
    }
    sum += __shfl_xor_sync(0xffffffffu, sum, 1);
    sum += __shfl_xor_sync(0xffffffffu, sum, 2);
    l = l * corr + sum;
    m = m_new;
    __syncwarp();
#pragma unroll
    for (int u = 0; u < WT_MAXD; ++u)
      if (u < nd) acc[u] *= corr;
    const float* pr = Ps + r * (WT_KEYS + 1);
    for (int kk = 0; kk < WT_KEYS; ++kk) {
      const float pj = pr[kk];
      const float* vr = Vs + kk * dvp;
#pragma unroll
      for (int u = 0; u < WT_MAXD; ++u) {
        const int d = c + 4 * u;
        if (u < nd && d < dv) acc[u] = fmaf(pj, vr[d], acc[u]);
      }
    }
  }
  if (!row_ok) return;
  const int t = row0 + r;
  const float inv = 1.f / l;
  CT* out = static_cast<CT*>(p.out) + static_cast<size_t>(t) * p.H * dv + h * dv;
  const float* gate = p.gate ? p.gate + static_cast<size_t>(t) * p.ld_gate + h * dv : nullptr;
#pragma unroll
  for (int u = 0; u < WT_MAXD; ++u) {
    const int d = c + 4 * u;
    if (u < nd && d < dv) {
      float o = acc[u] * inv;
      if (gate) o *= 1.f / (1.f + expf(-gate[d]));
      out[d] = wa_from_f<CT>(o);
    }
  }
}

// ------------------------------------------------------------------------------------------------------------------
// Decode rows: CTA = (token row, key/value head), 128 threads.  All R = H / G query heads of the group share every K / V
// tile of 32 positions, staged once in shared memory as fp32 with coalesced loads.  Warp w owns the heads r = w, w + 4, ..:
// lane j scores key j of the tile for them, the softmax statistics of a head stay inside its warp, and in the output phase
// lane d accumulates value dims d, d + 32, .. of the same heads.
// ------------------------------------------------------------------------------------------------------------------
constexpr int WD_KEYS = 32, WD_RU = 4, WD_VU = 8;      // up to 4 * WD_RU query heads per key/value head, vdim <= 32 * WD_VU

template <typename CT>
__global__ void __launch_bounds__(128) window_attn_group_kernel(WindowAttnParams p) {
  extern __shared__ float smf[];
  pdl_sync();
  const int t = blockIdx.x, g = blockIdx.y, R = p.H / p.G;
  const int dk = p.dim, dv = p.vdim, dkp = dk + 1, dvp = dv + 1;
  float* Qs = smf;                      // [R][dk]
  float* Ks = Qs + R * dk;              // [32][dk + 1]
  float* Vs = Ks + WD_KEYS * dkp;       // [32][dv + 1]
  float* Ps = Vs + WD_KEYS * dvp;       // [R][32]
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const CT* q = static_cast<const CT*>(p.q) + (static_cast<size_t>(t) * p.H + g * R) * dk;
  for (int i = tid; i < R * dk; i += 128) Qs[i] = wa_to_f(q[i]) * p.scale;
  const int b = p.row_req[t], ps = p.pos[t];
  const int32_t* pages = p.page_indices + p.page_indptr[b];
  const int lo = p.window > 0 ? max(0, ps - p.window + 1) : 0;
  const CT* kc = static_cast<const CT*>(p.k_cache);
  const CT* vc = static_cast<const CT*>(p.v_cache);
  float m[WD_RU], l[WD_RU], acc[WD_RU][WD_VU];
#pragma unroll
  for (int u = 0; u < WD_RU; ++u) {
    m[u] = -INFINITY;
    l[u] = 0.f;
#pragma unroll
    for (int v = 0; v < WD_VU; ++v) acc[u][v] = 0.f;
  }
  for (int c0 = lo; c0 <= ps; c0 += WD_KEYS) {
    __syncthreads();
    const int nk = min(WD_KEYS, ps - c0 + 1);
    for (int i = tid; i < WD_KEYS * dk; i += 128) {
      const int kk = i / dk, d = i - kk * dk;
      float v = 0.f;
      if (kk < nk) {
        const int kj = c0 + kk;
        const size_t tok = static_cast<size_t>(pages[kj / p.page_size]) * p.page_size + kj % p.page_size;
        v = wa_to_f(kc[(tok * p.G + g) * dk + d]);
      }
      Ks[kk * dkp + d] = v;
    }
    for (int i = tid; i < WD_KEYS * dv; i += 128) {
      const int kk = i / dv, d = i - kk * dv;
      float v = 0.f;
      if (kk < nk) {
        const int kj = c0 + kk;
        const size_t tok = static_cast<size_t>(pages[kj / p.page_size]) * p.page_size + kj % p.page_size;
        v = wa_to_f(vc[(tok * p.G + g) * dv + d]);
      }
      Vs[kk * dvp + d] = v;
    }
    __syncthreads();
#pragma unroll
    for (int u = 0; u < WD_RU; ++u) {
      const int r = warp + 4 * u;
      if (r >= R) break;
      float s = -INFINITY;
      if (lane < nk) {
        const float* qr = Qs + r * dk;
        const float* kr = Ks + lane * dkp;
        float a = 0.f;
        for (int d = 0; d < dk; ++d) a = fmaf(qr[d], kr[d], a);
        s = a;
      }
      const float m_new = fmaxf(m[u], warp_max(s));
      const float corr = expf(m[u] - m_new);
      const float pj = lane < nk ? expf(s - m_new) : 0.f;
      l[u] = l[u] * corr + warp_sum(pj);
      m[u] = m_new;
      Ps[r * WD_KEYS + lane] = pj;
      __syncwarp();
      const float* pr = Ps + r * WD_KEYS;
#pragma unroll
      for (int v = 0; v < WD_VU; ++v) {
        const int d = lane + 32 * v;
        if (d < dv) {
          float a = acc[u][v] * corr;
          for (int kk = 0; kk < nk; ++kk) a = fmaf(pr[kk], Vs[kk * dvp + d], a);
          acc[u][v] = a;
        }
      }
    }
  }
#pragma unroll
  for (int u = 0; u < WD_RU; ++u) {
    const int r = warp + 4 * u;
    if (r >= R) break;
    const int h = g * R + r;
    const float inv = 1.f / l[u];
    CT* out = static_cast<CT*>(p.out) + static_cast<size_t>(t) * p.H * dv + h * dv;
    const float* gate = p.gate ? p.gate + static_cast<size_t>(t) * p.ld_gate + h * dv : nullptr;
#pragma unroll
    for (int v = 0; v < WD_VU; ++v) {
      const int d = lane + 32 * v;
      if (d < dv) {
        float o = acc[u][v] * inv;
        if (gate) o *= 1.f / (1.f + expf(-gate[d]));
        out[d] = wa_from_f<CT>(o);
      }
    }
  }
}

}  // namespace vb

using namespace vb;
using bf16 = __nv_bfloat16;

extern "C" {

int vb_rotary_table(float* d_cs, const int32_t* d_pos, const double* d_freq, int T, int half, void* stream) {
  VB_CHECK_ARG(d_cs && d_pos && d_freq && half > 0, "vb_rotary_table: bad arguments");
  if (T <= 0) return 0;
  VB_LAUNCH_PDL(rotary_table_kernel, (T * half + 255) / 256, 256, 0, stream, d_cs, d_pos, d_freq, T, half);
  return 0;
}

int vb_qkv_rotary_append(const float* d_proj, int ldp, int q_off, int k_off, int v_off, const float* d_cs, int half,
                         void* d_q_out, void* d_k_cache, void* d_v_cache, const int32_t* d_row_req, const int32_t* d_pos,
                         const int32_t* d_page_indptr, const int32_t* d_page_indices, int page_size, int T, int H, int G,
                         int dim, int vdim, int vmix, float* d_v_first, const float* d_lambda, int dtype, void* stream) {
  VB_CHECK_ARG(d_proj && d_q_out && d_k_cache && d_v_cache && d_row_req && d_pos && d_page_indptr && d_page_indices,
               "vb_qkv_rotary_append: null pointer");
  VB_CHECK_ARG(H > 0 && G > 0 && H % G == 0 && dim > 0 && vdim > 0 && page_size > 0 && 2 * half <= dim,
               "vb_qkv_rotary_append: bad sizes H=%d G=%d dim=%d vdim=%d rotated=%d", H, G, dim, vdim, 2 * half);
  VB_CHECK_ARG(vmix == 0 || d_v_first, "vb_qkv_rotary_append: value mixing needs the first layer's values");
  VB_CHECK_ARG(vmix != 2 || d_lambda, "vb_qkv_rotary_append: value mixing needs its coefficient");
  if (T <= 0) return 0;
  QkvTailParams p{d_proj, ldp, q_off, k_off, v_off, half > 0 ? d_cs : nullptr, half, d_q_out, d_k_cache, d_v_cache,
                  d_row_req, d_pos, d_page_indptr, d_page_indices, page_size, H, G, dim, vdim, vmix, d_v_first, d_lambda};
  if (dtype == 1) VB_LAUNCH_PDL(qkv_rotary_append_kernel<float>, T, 256, 0, stream, p);
  else VB_LAUNCH_PDL(qkv_rotary_append_kernel<bf16>, T, 256, 0, stream, p);
  return 0;
}

int vb_window_attn(void* d_out, const void* d_q, const void* d_k_cache, const void* d_v_cache, const float* d_gate,
                   int ld_gate, const int32_t* d_row_req, const int32_t* d_pos, const int32_t* d_page_indptr,
                   const int32_t* d_page_indices, int T, int H, int G, int dim, int vdim, int page_size, int window,
                   float scale, int dtype, void* stream) {
  VB_CHECK_ARG(d_out && d_q && d_k_cache && d_v_cache && d_row_req && d_pos && d_page_indptr && d_page_indices,
               "vb_window_attn: null pointer");
  VB_CHECK_ARG(H > 0 && G > 0 && H % G == 0 && dim > 0 && vdim > 0 && vdim <= 32 * WA_MAXU && page_size > 0,
               "vb_window_attn: bad sizes H=%d G=%d dim=%d vdim=%d (vdim <= %d)", H, G, dim, vdim, 32 * WA_MAXU);
  if (T <= 0) return 0;
  WindowAttnParams p{d_q, d_k_cache, d_v_cache, d_out, d_gate, ld_gate, d_row_req, d_pos, d_page_indptr, d_page_indices,
                     nullptr, nullptr, nullptr, T, H, G, dim, vdim, page_size, window, scale};
  // a CTA per (row, key/value head) with the K / V tiles shared by the group's query heads, when the group fits its
  // registers and the tiles fit shared memory; one warp per (row, query head) otherwise
  const int R = H / G;
  const size_t gsmem = (static_cast<size_t>(R) * dim + static_cast<size_t>(WD_KEYS) * (dim + 1 + vdim + 1) +
                        static_cast<size_t>(R) * WD_KEYS) * sizeof(float);
  if (R <= 4 * WD_RU && vdim <= 32 * WD_VU && gsmem <= 96 * 1024) {
    dim3 ggrid(T, G);
    if (dtype == 1) {
      VB_CHECK_CUDA(cudaFuncSetAttribute(window_attn_group_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, VB_MAX_DYN_SMEM));
      VB_LAUNCH_PDL(window_attn_group_kernel<float>, ggrid, 128, gsmem, stream, p);
    } else {
      VB_CHECK_CUDA(cudaFuncSetAttribute(window_attn_group_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, VB_MAX_DYN_SMEM));
      VB_LAUNCH_PDL(window_attn_group_kernel<bf16>, ggrid, 128, gsmem, stream, p);
    }
    return 0;
  }
  const size_t smem = static_cast<size_t>(WA_WARPS) * dim * sizeof(float);
  VB_CHECK_ARG(smem <= 48 * 1024, "vb_window_attn: head dim %d too large", dim);
  dim3 grid((T + WA_WARPS - 1) / WA_WARPS, H);
  if (dtype == 1) VB_LAUNCH_PDL(window_attn_kernel<float>, grid, WA_WARPS * 32, smem, stream, p);
  else VB_LAUNCH_PDL(window_attn_kernel<bf16>, grid, WA_WARPS * 32, smem, stream, p);
  return 0;
}

int vb_window_attn_tile_rows(void) { return WT_ROWS; }

int vb_window_attn_tiled(void* d_out, const void* d_q, const void* d_k_cache, const void* d_v_cache, const float* d_gate,
                         int ld_gate, const int32_t* d_pos, const int32_t* d_page_indptr, const int32_t* d_page_indices,
                         const int32_t* d_qo_indptr, const int32_t* d_tile_req, const int32_t* d_tile_row0, int n_tiles,
                         int T, int H, int G, int dim, int vdim, int page_size, int window, float scale, int dtype,
                         void* stream) {
  VB_CHECK_ARG(d_out && d_q && d_k_cache && d_v_cache && d_pos && d_page_indptr && d_page_indices && d_qo_indptr &&
               d_tile_req && d_tile_row0, "vb_window_attn_tiled: null pointer");
  VB_CHECK_ARG(H > 0 && G > 0 && H % G == 0 && dim > 0 && vdim > 0 && vdim <= 4 * WT_MAXD && page_size > 0,
               "vb_window_attn_tiled: bad sizes H=%d G=%d dim=%d vdim=%d", H, G, dim, vdim);
  if (n_tiles <= 0) return 0;
  WindowAttnParams p{d_q, d_k_cache, d_v_cache, d_out, d_gate, ld_gate, nullptr, d_pos, d_page_indptr, d_page_indices,
                     d_qo_indptr, d_tile_req, d_tile_row0, T, H, G, dim, vdim, page_size, window, scale};
  const size_t smem = (static_cast<size_t>(WT_ROWS + WT_KEYS) * (dim + 1) + static_cast<size_t>(WT_KEYS) * (vdim + 1) +
                       static_cast<size_t>(WT_ROWS) * (WT_KEYS + 1)) * sizeof(float);
  VB_CHECK_ARG(smem <= static_cast<size_t>(VB_MAX_DYN_SMEM), "vb_window_attn_tiled: heads too large for shared memory");
  dim3 grid(n_tiles, H);
  if (dtype == 1) {
    VB_CHECK_CUDA(cudaFuncSetAttribute(window_attn_tiled_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, VB_MAX_DYN_SMEM));
    VB_LAUNCH_PDL(window_attn_tiled_kernel<float>, grid, 256, smem, stream, p);
  } else {
    VB_CHECK_CUDA(cudaFuncSetAttribute(window_attn_tiled_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, VB_MAX_DYN_SMEM));
    VB_LAUNCH_PDL(window_attn_tiled_kernel<bf16>, grid, 256, smem, stream, p);
  }
  return 0;
}

}  // extern "C"
