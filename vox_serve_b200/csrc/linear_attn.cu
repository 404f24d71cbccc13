// Linear attention with a per-head scalar decay ("lightning" attention): per head the state S [dim][vdim] follows
//   S_t = decay * S_(t-1) + k_t v_t^T,      o_t = S_t^T q_t
// with q, k, v = silu of a fused projection's columns.  The state lives in fp32 in a slot per live sequence and is
// carried from step to step; everything after the projection is fp32.
//
//   vb_decay_attn_chunked   prompt portions.  CTA = (request, head, block of value dims).  The portion is walked in chunks
//                           of C tokens: scores A = (Q K^T) .* decay^(i-j) for j <= i, output O = A V + decay^(i+1) Q S,
//                           then S <- decay^C S + sum_j decay^(C-1-j) k_j v_j^T.  Only non-negative powers of the decay
//                           appear, so small decays underflow to zero instead of overflowing.
//   vb_decay_attn_tiled     the same result with the portion's chunks processed in parallel (local chunk states, a scan over
//                           them, outputs per chunk): what a long prompt runs
//   vb_decay_attn_step      single new tokens: CTA = (request, head, block of value dims), one read and one write of the
//                           state, the output reduced over the key dims in shared memory.
//   vb_gated_rmsnorm        rows of concatenated heads: x / sqrt(mean(x^2) + eps) * weight * sigmoid(gate).
// A request whose first new token has position 0 starts from a zero state (the slot's old content is not read).
#include "../../include/vb_api.h"
#define VB_PDL_FAMILY 1
#include "common.cuh"

namespace vb {

__device__ __forceinline__ float silu_f(float z) { return z / (1.f + expf(-z)); }

struct DecayAttnParams {
  const float* proj;         // [T][ldp]
  int ldp, q_off, k_off, v_off;
  float* out;                // [T][H * vdim]
  float* state;              // [slots][H][dim][vdim]
  const float* decay;        // [H]
  const int32_t* qo_indptr;  // [B + 1]
  const int32_t* pos;        // [T]
  const int32_t* slots;      // [B]
  int H, dim, vdim, dvb, chunk, min_rows, max_rows;   // requests with min_rows <= new rows <= max_rows are served
};

__global__ void __launch_bounds__(256) decay_attn_chunked_kernel(DecayAttnParams p) {
  extern __shared__ float smf[];
  pdl_sync();
  const int b = blockIdx.x, h = blockIdx.y, e0 = blockIdx.z * p.dvb;
  const int r0 = p.qo_indptr[b], n = p.qo_indptr[b + 1] - r0;
  if (n < p.min_rows || n > p.max_rows) return;
  const int C = p.chunk, dk = p.dim, dkp = dk + 1, DV = min(p.dvb, p.vdim - e0);
  const int dvp = p.dvb + 1;
  float* Sq = smf;                    // [C][dk + 1]
  float* Sk = Sq + C * dkp;           // [C][dk + 1]
  float* Sv = Sk + C * dkp;           // [C][dvb + 1]
  float* Sa = Sv + C * dvp;           // [C][C + 1]
  float* Ss = Sa + C * (C + 1);       // [dk][dvb + 1]
  float* pw = Ss + dk * dvp;          // [C + 1] powers of the decay
  const int tid = threadIdx.x;
  const double d = static_cast<double>(p.decay[h]);
  for (int i = tid; i <= C; i += 256) pw[i] = static_cast<float>(pow(d, static_cast<double>(i)));
  float* S = p.state + ((static_cast<size_t>(p.slots[b]) * p.H + h) * dk) * p.vdim;
  const bool fresh = p.pos[r0] == 0;
  for (int i = tid; i < dk * DV; i += 256) {
    const int k = i / DV, e = i - k * DV;
    Ss[k * dvp + e] = fresh ? 0.f : S[static_cast<size_t>(k) * p.vdim + e0 + e];
  }
  for (int c0 = 0; c0 < n; c0 += C) {
    const int L = min(C, n - c0);
    __syncthreads();
    for (int i = tid; i < C * dk; i += 256) {
      const int r = i / dk, k = i - r * dk;
      float qv = 0.f, kv = 0.f;
      if (r < L) {
        const float* row = p.proj + static_cast<size_t>(r0 + c0 + r) * p.ldp + h * dk + k;
        qv = silu_f(row[p.q_off]);
        kv = silu_f(row[p.k_off]);
      }
      Sq[r * dkp + k] = qv;
      Sk[r * dkp + k] = kv;
    }
    for (int i = tid; i < C * DV; i += 256) {
      const int r = i / DV, e = i - r * DV;
      Sv[r * dvp + e] = r < L ? silu_f(p.proj[static_cast<size_t>(r0 + c0 + r) * p.ldp + p.v_off + h * p.vdim + e0 + e]) : 0.f;
    }
    __syncthreads();
    for (int i = tid; i < C * C; i += 256) {
      const int r = i / C, j = i - r * C;
      float a = 0.f;
      if (j <= r && r < L) {
        const float* qr = Sq + r * dkp;
        const float* kr = Sk + j * dkp;
        for (int k = 0; k < dk; ++k) a = fmaf(qr[k], kr[k], a);
        a *= pw[r - j];
      }
      Sa[r * (C + 1) + j] = a;
    }
    __syncthreads();
    for (int i = tid; i < L * DV; i += 256) {
      const int r = i / DV, e = i - r * DV;
      float intra = 0.f, inter = 0.f;
      const float* ar = Sa + r * (C + 1);
      for (int j = 0; j <= r; ++j) intra = fmaf(ar[j], Sv[j * dvp + e], intra);
      const float* qr = Sq + r * dkp;
      for (int k = 0; k < dk; ++k) inter = fmaf(qr[k], Ss[k * dvp + e], inter);
      p.out[static_cast<size_t>(r0 + c0 + r) * p.H * p.vdim + h * p.vdim + e0 + e] = intra + pw[r + 1] * inter;
    }
    __syncthreads();
    const float dl = pw[L];
    for (int i = tid; i < dk * DV; i += 256) {
      const int k = i / DV, e = i - k * DV;
      float a = 0.f;
      for (int j = 0; j < L; ++j) a = fmaf(pw[L - 1 - j] * Sk[j * dkp + k], Sv[j * dvp + e], a);
      Ss[k * dvp + e] = dl * Ss[k * dvp + e] + a;
    }
  }
  __syncthreads();
  for (int i = tid; i < dk * DV; i += 256) {
    const int k = i / DV, e = i - k * DV;
    S[static_cast<size_t>(k) * p.vdim + e0 + e] = Ss[k * dvp + e];
  }
}

// one new token per request: threads = (key group kg, value dim e); the key dims are strided over the groups
__global__ void __launch_bounds__(256) decay_attn_step_kernel(DecayAttnParams p) {
  extern __shared__ float smf[];
  pdl_sync();
  const int b = blockIdx.x, h = blockIdx.y, e0 = blockIdx.z * p.dvb;
  const int r0 = p.qo_indptr[b], n = p.qo_indptr[b + 1] - r0;
  if (n < p.min_rows || n > p.max_rows) return;
  const int dk = p.dim, DV = min(p.dvb, p.vdim - e0);
  float* qs = smf;              // [dk]
  float* ks = qs + dk;          // [dk]
  float* red = ks + dk;         // [groups][dvb]
  const int tid = threadIdx.x, groups = 256 / p.dvb, e = tid % p.dvb, kg = tid / p.dvb;
  const float dec = p.decay[h];
  float* S = p.state + ((static_cast<size_t>(p.slots[b]) * p.H + h) * dk) * p.vdim;
  for (int r = 0; r < n; ++r) {
    const float* row = p.proj + static_cast<size_t>(r0 + r) * p.ldp;
    const bool fresh = p.pos[r0 + r] == 0;
    __syncthreads();
    for (int k = tid; k < dk; k += 256) {
      qs[k] = silu_f(row[p.q_off + h * dk + k]);
      ks[k] = silu_f(row[p.k_off + h * dk + k]);
    }
    __syncthreads();
    float o = 0.f;
    if (e < DV && kg < groups) {
      const float v = silu_f(row[p.v_off + h * p.vdim + e0 + e]);
      for (int k = kg; k < dk; k += groups) {
        float* sp = S + static_cast<size_t>(k) * p.vdim + e0 + e;
        const float s = (fresh ? 0.f : dec * *sp) + ks[k] * v;
        *sp = s;
        o = fmaf(s, qs[k], o);
      }
    }
    if (kg < groups) red[kg * p.dvb + e] = o;
    __syncthreads();
    if (tid < DV) {
      float t = 0.f;
      for (int gI = 0; gI < groups; ++gI) t += red[gI * p.dvb + tid];
      p.out[static_cast<size_t>(r0 + r) * p.H * p.vdim + h * p.vdim + e0 + tid] = t;
    }
  }
}


// ------------------------------------------------------------------------------------------------------------------
// Sequence-parallel form for prompt portions.  The portion of every request is cut into tiles of DT_ROWS consecutive rows
// (tile i = rows tile_row0[i].. of request tile_req[i]; the tiles of a request are consecutive, requests in batch order,
// only requests that bring two or more rows have tiles):
//   1. per tile, in parallel:  U = sum_j decay^(L-1-j) k_j v_j^T                      -> scratch[tile][h]
//   2. per request, in order:  scratch[tile][h] <- S before the tile;  S <- decay^L S + U;  the slot gets the final S
//   3. per tile, in parallel:  O = (Q K^T .* decay^(i-j), j <= i) V + decay^(i+1) Q S_before
// ------------------------------------------------------------------------------------------------------------------
constexpr int DT_ROWS = 64;

struct DecayTileParams {
  DecayAttnParams a;
  float* scratch;              // [tiles][H][dim][vdim]
  const int32_t* tile_req;
  const int32_t* tile_row0;
  int B;
};

__global__ void __launch_bounds__(256) decay_tile_state_kernel(DecayTileParams tp) {
  extern __shared__ float smf[];
  pdl_sync();
  const DecayAttnParams& p = tp.a;
  const int tile = blockIdx.x, h = blockIdx.y, e0 = blockIdx.z * p.dvb;
  const int b = tp.tile_req[tile], row0 = tp.tile_row0[tile];
  const int L = min(DT_ROWS, p.qo_indptr[b + 1] - row0);
  const int dk = p.dim, dkp = dk + 1, DV = min(p.dvb, p.vdim - e0), dvp = p.dvb + 1;
  float* Sk = smf;                       // [64][dk + 1]
  float* Sv = Sk + DT_ROWS * dkp;        // [64][dvb + 1]
  float* pw = Sv + DT_ROWS * dvp;        // [65]
  const int tid = threadIdx.x;
  const double d = static_cast<double>(p.decay[h]);
  for (int i = tid; i <= DT_ROWS; i += 256) pw[i] = static_cast<float>(pow(d, static_cast<double>(i)));
  for (int i = tid; i < L * dk; i += 256) {
    const int r = i / dk, k = i - r * dk;
    Sk[r * dkp + k] = silu_f(p.proj[static_cast<size_t>(row0 + r) * p.ldp + p.k_off + h * dk + k]);
  }
  for (int i = tid; i < L * DV; i += 256) {
    const int r = i / DV, e = i - r * DV;
    Sv[r * dvp + e] = silu_f(p.proj[static_cast<size_t>(row0 + r) * p.ldp + p.v_off + h * p.vdim + e0 + e]);
  }
  __syncthreads();
  float* U = tp.scratch + ((static_cast<size_t>(tile) * p.H + h) * dk) * p.vdim;
  // register tiles: thread (ty, tx) owns key dims ty + 16 i and value dims tx + 16 e; per position it reads its key values
  // (two distinct rows of addresses per warp: broadcast) and value values (consecutive addresses) once for 32 FMAs
  const int tx = tid & 15, ty = tid >> 4;
  for (int kb = 0; kb < dk; kb += 128) {
    float acc[8][4];
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
      for (int e = 0; e < 4; ++e) acc[i][e] = 0.f;
    for (int j = 0; j < L; ++j) {
      const float w = pw[L - 1 - j];
      float kv[8], vv[4];
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int k = kb + ty + 16 * i;
        kv[i] = k < dk ? Sk[j * dkp + k] : 0.f;
      }
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int ee = tx + 16 * e;
        vv[e] = ee < DV ? w * Sv[j * dvp + ee] : 0.f;
      }
#pragma unroll
      for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int e = 0; e < 4; ++e) acc[i][e] = fmaf(kv[i], vv[e], acc[i][e]);
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int k = kb + ty + 16 * i;
      if (k >= dk) continue;
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int ee = tx + 16 * e;
        if (ee < DV) U[static_cast<size_t>(k) * p.vdim + e0 + ee] = acc[i][e];
      }
    }
  }
}

__global__ void __launch_bounds__(256) decay_tile_scan_kernel(DecayTileParams tp) {
  pdl_sync();
  const DecayAttnParams& p = tp.a;
  const int b = blockIdx.x, h = blockIdx.y;
  const int r0 = p.qo_indptr[b], n = p.qo_indptr[b + 1] - r0;
  if (n < 2) return;
  int first = 0;                          // tiles of the requests before this one
  for (int bb = 0; bb < b; ++bb) {
    const int nn = p.qo_indptr[bb + 1] - p.qo_indptr[bb];
    if (nn >= 2) first += (nn + DT_ROWS - 1) / DT_ROWS;
  }
  const int n_tiles = (n + DT_ROWS - 1) / DT_ROWS;
  const bool fresh = p.pos[r0] == 0;
  const double d = static_cast<double>(p.decay[h]);
  const float d_full = static_cast<float>(pow(d, static_cast<double>(DT_ROWS)));
  const float d_last = static_cast<float>(pow(d, static_cast<double>(n - (n_tiles - 1) * DT_ROWS)));
  const size_t per = static_cast<size_t>(p.dim) * p.vdim;
  float* S = p.state + (static_cast<size_t>(p.slots[b]) * p.H + h) * per;
  for (size_t i = blockIdx.z * blockDim.x + threadIdx.x; i < per; i += static_cast<size_t>(gridDim.z) * blockDim.x) {
    float s = fresh ? 0.f : S[i];
    for (int c0 = 0; c0 < n_tiles; c0 += 8) {          // eight independent loads in flight, then the serial update
      float uv[8];
#pragma unroll
      for (int j = 0; j < 8; ++j)
        uv[j] = c0 + j < n_tiles ? tp.scratch[(static_cast<size_t>(first + c0 + j) * p.H + h) * per + i] : 0.f;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int c = c0 + j;
        if (c < n_tiles) {
          tp.scratch[(static_cast<size_t>(first + c) * p.H + h) * per + i] = s;
          s = (c == n_tiles - 1 ? d_last : d_full) * s + uv[j];
        }
      }
    }
    S[i] = s;
  }
}

__global__ void __launch_bounds__(256) decay_tile_out_kernel(DecayTileParams tp) {
  extern __shared__ float smf[];
  pdl_sync();
  const DecayAttnParams& p = tp.a;
  const int tile = blockIdx.x, h = blockIdx.y, e0 = blockIdx.z * p.dvb;
  const int b = tp.tile_req[tile], row0 = tp.tile_row0[tile];
  const int L = min(DT_ROWS, p.qo_indptr[b + 1] - row0);
  constexpr int C = DT_ROWS;
  // shared memory is laid out for two CTAs per SM at 128-wide heads: the scores overwrite the key tile once it has been
  // consumed, and the value / state tiles (read along the value dim only) carry no padding
  const int dk = p.dim, dkp = dk + 1, DV = min(p.dvb, p.vdim - e0), dvp = p.dvb;
  float* Sq = smf;                                   // [C][dk + 1]
  float* Sk = Sq + C * dkp;                          // [C][dk + 1], then the scores [C][C + 1]
  float* Sa = Sk;
  float* Sv = Sk + C * max(dkp, C + 1);              // [C][dvb]
  float* Ss = Sv + C * dvp;                          // [dk][dvb]
  float* pw = Ss + dk * dvp;                         // [C + 1]
  const int tid = threadIdx.x;
  const double d = static_cast<double>(p.decay[h]);
  for (int i = tid; i <= C; i += 256) pw[i] = static_cast<float>(pow(d, static_cast<double>(i)));
  const float* Sb = tp.scratch + ((static_cast<size_t>(tile) * p.H + h) * dk) * p.vdim;
  for (int i = tid; i < dk * DV; i += 256) {
    const int k = i / DV, e = i - k * DV;
    Ss[k * dvp + e] = Sb[static_cast<size_t>(k) * p.vdim + e0 + e];
  }
  for (int i = tid; i < C * dk; i += 256) {
    const int r = i / dk, k = i - r * dk;
    float qv = 0.f, kv = 0.f;
    if (r < L) {
      const float* row = p.proj + static_cast<size_t>(row0 + r) * p.ldp + h * dk + k;
      qv = silu_f(row[p.q_off]);
      kv = silu_f(row[p.k_off]);
    }
    Sq[r * dkp + k] = qv;
    Sk[r * dkp + k] = kv;
  }
  for (int i = tid; i < C * DV; i += 256) {
    const int r = i / DV, e = i - r * DV;
    Sv[r * dvp + e] = r < L ? silu_f(p.proj[static_cast<size_t>(row0 + r) * p.ldp + p.v_off + h * p.vdim + e0 + e]) : 0.f;
  }
  __syncthreads();
  // register tiles (C = 64, 16 x 16 threads): thread (ty, tx) owns rows ty + 16 i and columns tx + 16 j
  const int tx = tid & 15, ty = tid >> 4;
  {
    float a[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) a[i][j] = 0.f;
    for (int k = 0; k < dk; ++k) {
      float qv[4], kv[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) qv[i] = Sq[(ty + 16 * i) * dkp + k];
#pragma unroll
      for (int j = 0; j < 4; ++j) kv[j] = Sk[(tx + 16 * j) * dkp + k];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) a[i][j] = fmaf(qv[i], kv[j], a[i][j]);
    }
    __syncthreads();                                 // the key tile is consumed: its place takes the scores
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int r = ty + 16 * i, c = tx + 16 * j;
        Sa[r * (C + 1) + c] = (c <= r && r < L) ? a[i][j] * pw[r - c] : 0.f;
      }
  }
  __syncthreads();
  {
    float intra[4][4], inter[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int e = 0; e < 4; ++e) intra[i][e] = inter[i][e] = 0.f;
    const int jmax = min(L, ty + 49);              // the thread's last row is ty + 48: later positions are masked for all
    for (int j = 0; j < jmax; ++j) {
      float av[4], vv[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) av[i] = Sa[(ty + 16 * i) * (C + 1) + j];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int ee = tx + 16 * e;
        vv[e] = ee < DV ? Sv[j * dvp + ee] : 0.f;
      }
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int e = 0; e < 4; ++e) intra[i][e] = fmaf(av[i], vv[e], intra[i][e]);
    }
    for (int k = 0; k < dk; ++k) {
      float qv[4], sv[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) qv[i] = Sq[(ty + 16 * i) * dkp + k];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int ee = tx + 16 * e;
        sv[e] = ee < DV ? Ss[k * dvp + ee] : 0.f;
      }
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int e = 0; e < 4; ++e) inter[i][e] = fmaf(qv[i], sv[e], inter[i][e]);
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int r = ty + 16 * i;
      if (r >= L) continue;
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int ee = tx + 16 * e;
        if (ee < DV)
          p.out[static_cast<size_t>(row0 + r) * p.H * p.vdim + h * p.vdim + e0 + ee] = intra[i][e] + pw[r + 1] * inter[i][e];
      }
    }
  }
}

template <typename OT>
__global__ void gated_rmsnorm_kernel(OT* __restrict__ out, const float* __restrict__ x, const float* __restrict__ w,
                                     const float* __restrict__ gate, int ld_gate, int N, float eps) {
  __shared__ float red[40];
  pdl_sync();
  const size_t t = blockIdx.x;
  const float* row = x + t * N;
  float q = 0.f;
  for (int i = threadIdx.x; i < N; i += blockDim.x) q += row[i] * row[i];
  const int lane = threadIdx.x & 31, wp = threadIdx.x >> 5;
  q = warp_sum(q);
  if (lane == 0) red[wp] = q;
  __syncthreads();
  if (wp == 0) {
    float s = lane < (blockDim.x >> 5) ? red[lane] : 0.f;
    s = warp_sum(s);
    if (lane == 0) red[32] = s;
  }
  __syncthreads();
  const float rstd = 1.f / sqrtf(red[32] / N + eps);
  for (int i = threadIdx.x; i < N; i += blockDim.x) {
    float v = row[i] * rstd * w[i];
    if (gate) v *= 1.f / (1.f + expf(-gate[t * ld_gate + i]));
    if constexpr (sizeof(OT) == 4) out[t * N + i] = v;
    else out[t * N + i] = __float2bfloat16_rn(v);
  }
}

static size_t chunked_smem(int C, int dk, int dvb) {
  return (2ull * C * (dk + 1) + static_cast<size_t>(C) * (dvb + 1) + static_cast<size_t>(C) * (C + 1) +
          static_cast<size_t>(dk) * (dvb + 1) + C + 1) * sizeof(float);
}

static int decay_dvb(int vdim) {
  int dvb = 64;
  while (dvb > 1 && dvb / 2 >= vdim) dvb /= 2;       // the smallest power of two >= vdim, at most 64
  return dvb;
}

}  // namespace vb

using namespace vb;

extern "C" {

int vb_decay_attn(float* d_out, float* d_state, const float* d_proj, int ldp, int q_off, int k_off, int v_off,
                  const float* d_decay, const int32_t* d_qo_indptr, const int32_t* d_pos, const int32_t* d_slots, int B,
                  int H, int dim, int vdim, int single_rows, int multi_rows, void* stream) {
  VB_CHECK_ARG(d_out && d_state && d_proj && d_decay && d_qo_indptr && d_pos && d_slots, "vb_decay_attn: null pointer");
  VB_CHECK_ARG(H > 0 && dim > 0 && vdim > 0, "vb_decay_attn: bad sizes H=%d dim=%d vdim=%d", H, dim, vdim);
  if (B <= 0) return 0;
  const int dvb = decay_dvb(vdim);
  DecayAttnParams p{d_proj, ldp, q_off, k_off, v_off, d_out, d_state, d_decay, d_qo_indptr, d_pos, d_slots,
                    H, dim, vdim, dvb, 0, 0, 0};
  dim3 grid(B, H, (vdim + dvb - 1) / dvb);
  if (single_rows) {          // requests that bring exactly one token
    p.min_rows = 1;
    p.max_rows = 1;
    const size_t smem = (2ull * dim + 256) * sizeof(float);
    VB_CHECK_ARG(smem <= 48 * 1024, "vb_decay_attn: head dim %d too large", dim);
    VB_LAUNCH_PDL(decay_attn_step_kernel, grid, 256, smem, stream, p);
  }
  if (multi_rows) {           // requests that bring a portion of a prompt
    p.min_rows = 2;
    p.max_rows = 1 << 30;
    int C = 64;
    while (C > 8 && chunked_smem(C, dim, dvb) > 200 * 1024) C /= 2;
    const size_t smem = chunked_smem(C, dim, dvb);
    VB_CHECK_ARG(smem <= static_cast<size_t>(VB_MAX_DYN_SMEM), "vb_decay_attn: head dim %d too large", dim);
    p.chunk = C;
    VB_CHECK_CUDA(cudaFuncSetAttribute(decay_attn_chunked_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, VB_MAX_DYN_SMEM));
    VB_LAUNCH_PDL(decay_attn_chunked_kernel, grid, 256, smem, stream, p);
  }
  return 0;
}

/* rows per tile of the sequence-parallel form, or 0 when these head sizes do not fit its shared memory */
int vb_decay_attn_tile_rows(int dim, int vdim) {
  return chunked_smem(DT_ROWS, dim, decay_dvb(vdim)) <= static_cast<size_t>(VB_MAX_DYN_SMEM) ? DT_ROWS : 0;
}

int vb_decay_attn_tiled(float* d_out, float* d_state, float* d_scratch, const float* d_proj, int ldp, int q_off, int k_off,
                        int v_off, const float* d_decay, const int32_t* d_qo_indptr, const int32_t* d_pos,
                        const int32_t* d_slots, const int32_t* d_tile_req, const int32_t* d_tile_row0, int n_tiles, int B,
                        int H, int dim, int vdim, void* stream) {
  VB_CHECK_ARG(d_out && d_state && d_scratch && d_proj && d_decay && d_qo_indptr && d_pos && d_slots && d_tile_req &&
               d_tile_row0, "vb_decay_attn_tiled: null pointer");
  VB_CHECK_ARG(H > 0 && dim > 0 && vdim > 0 && vb_decay_attn_tile_rows(dim, vdim) > 0, "vb_decay_attn_tiled: bad sizes");
  if (n_tiles <= 0 || B <= 0) return 0;
  const int dvb = decay_dvb(vdim);
  DecayTileParams tp{{d_proj, ldp, q_off, k_off, v_off, d_out, d_state, d_decay, d_qo_indptr, d_pos, d_slots, H, dim, vdim,
                      dvb, DT_ROWS, 2, 1 << 30}, d_scratch, d_tile_req, d_tile_row0, B};
  const int zb = (vdim + dvb - 1) / dvb;
  const size_t smem1 = (static_cast<size_t>(DT_ROWS) * (dim + 1 + dvb + 1) + DT_ROWS + 1) * sizeof(float);
  const size_t smem3 = (static_cast<size_t>(DT_ROWS) * (dim + 1) + static_cast<size_t>(DT_ROWS) * max(dim + 1, DT_ROWS + 1) +
                        static_cast<size_t>(DT_ROWS) * dvb + static_cast<size_t>(dim) * dvb + DT_ROWS + 1) * sizeof(float);
  VB_CHECK_CUDA(cudaFuncSetAttribute(decay_tile_state_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, VB_MAX_DYN_SMEM));
  VB_CHECK_CUDA(cudaFuncSetAttribute(decay_tile_out_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, VB_MAX_DYN_SMEM));
  VB_LAUNCH_PDL(decay_tile_state_kernel, dim3(n_tiles, H, zb), 256, smem1, stream, tp);
  const size_t per = static_cast<size_t>(dim) * vdim;
  VB_LAUNCH_PDL(decay_tile_scan_kernel, dim3(B, H, static_cast<unsigned>((per + 1023) / 1024)), 256, 0, stream, tp);
  VB_LAUNCH_PDL(decay_tile_out_kernel, dim3(n_tiles, H, zb), 256, smem3, stream, tp);
  return 0;
}

int vb_gated_rmsnorm(void* d_out, const float* d_x, const float* d_w, const float* d_gate, int ld_gate, int T, int N,
                     float eps, int out_dtype, void* stream) {
  VB_CHECK_ARG(d_out && d_x && d_w && N > 0, "vb_gated_rmsnorm: bad arguments");
  if (T <= 0) return 0;
  if (out_dtype == 1) VB_LAUNCH_PDL(gated_rmsnorm_kernel<float>, T, 256, 0, stream, static_cast<float*>(d_out), d_x, d_w, d_gate, ld_gate, N, eps);
  else VB_LAUNCH_PDL(gated_rmsnorm_kernel<__nv_bfloat16>, T, 256, 0, stream, static_cast<__nv_bfloat16*>(d_out), d_x, d_w, d_gate, ld_gate, N, eps);
  return 0;
}

}  // extern "C"
