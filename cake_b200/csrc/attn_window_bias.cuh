// attn_window_bias.cuh — grouped-query attention with the score modifiers of the layer-list blocks (include/cake_b200.h,
// cake_b200_layer_spec), all of them parameters:
//
//   s_ij = (q_i . k_j) * scale
//   softcap > 0      s <- softcap * tanh(s / softcap)
//   r1, r2 non-null  s <- s - r1[h] * ln(1 + r2[h] * (i - j))           (a bias that grows with the distance, per query head)
//   window > 0       row i attends to the keys j with i - window < j <= i; window == 0: every j <= i
//   p = softmax over the visible j (fp32);   out_i = sum_j p_ij v_j   with v == k when the keys double as values (vc == kc)
//   gate_col >= 0    out_i <- out_i * sigmoid(z_ih), z_ih = column gate_col + h of the projection row of token i
//
// Scores, bias, softmax and the weighted sum are fp32 whatever D is.  Keys are read only from the cache (the step's own
// keys are appended before the launch), so a position's result does not depend on how the prompt was cut into steps.
// Kernels:
//   attn_window_bias_kernel      one warp per (token, head), any head_dim <= 256 and any D (float included): a lane scores
//                                one key of a 32-key tile, the tile's keys are then accumulated dimension-parallel
//   attn_window_decode_kernel    one CTA per (token, head) for steps of a few tokens: its warps split the window and merge
//                                their partial softmax states in shared memory
//   attn_window_decode_vec_kernel the same for 16-bit D with rows of whole 16-byte pieces and values == keys: eight lanes
//                                per key, the row read once for the score and the weighted sum
//   attn_window_mma_kernel       prompt portions on the tensor cores for 16-bit D (below)
// Nothing here follows a reference file: the reference has none of these modifiers.
#pragma once
#include "attn_prefill.cuh"
#include "common.cuh"
#include "f32_stream.cuh"

namespace cake {

struct WinAttn {
  const void *qkg;       // [B*S, ld] D: q of head h at columns [h*hd, (h+1)*hd); gate logits at gate_col + h
  const void *kc, *vc;   // [B, n_kv, cap, hd] D
  const void *r1, *r2;   // [heads] D or null
  void *y;               // [B*S, ldy] D: head h at columns [h*hd, (h+1)*hd)
  int B, S, heads, n_kv, hd, cap, pos0, ld, ldy, gate_col, window;
  float scale, softcap;
  // attn_window_tc_kernel only (zero = absent):
  int keep_first;        // keys [0, keep_first) stay visible to every later row, whatever the window
  int key0;              // the position of row 0 of kc / vc (a buffer that starts at the first key any row of the step sees)
  const void *sink;      // [heads] D: a logit that joins every row's denominator, without key or value
  const void *gate;      // gate_mode 1: [B*S, ldg] D logits, one per head at column h; 2: one per output element at h*hd + i
  int gate_mode, ldg;
};
constexpr int WA_MAX_HD = 256;

// q (fp32, shared memory) . k (D, global), 16-byte loads when the row allows them
template <typename T> __device__ __forceinline__ float wa_dot(const float *q, const T *k, int hd);
template <> __device__ __forceinline__ float wa_dot<float>(const float *q, const float *k, int hd) {
  float s = 0.f;
  if ((hd & 3) == 0) {
    const float4 *k4 = reinterpret_cast<const float4 *>(k);
    for (int i = 0; i < hd / 4; i++) {
      const float4 v = k4[i];
      s = fmaf(q[4 * i], v.x, s); s = fmaf(q[4 * i + 1], v.y, s); s = fmaf(q[4 * i + 2], v.z, s); s = fmaf(q[4 * i + 3], v.w, s);
    }
  } else
    for (int i = 0; i < hd; i++) s = fmaf(q[i], k[i], s);
  return s;
}
template <typename T> __device__ __forceinline__ float wa_dot(const float *q, const T *k, int hd) {
  float s = 0.f;
  if ((hd & 7) == 0) {
    const uint4 *k4 = reinterpret_cast<const uint4 *>(k);
    for (int i = 0; i < hd / 8; i++) {
      float f[8];
      unpack8<T>(k4[i], f);
#pragma unroll
      for (int e = 0; e < 8; e++) s = fmaf(q[8 * i + e], f[e], s);
    }
  } else
    for (int i = 0; i < hd; i++) s = fmaf(q[i], DT<T>::to_f(k[i]), s);
  return s;
}

// the modified score of query position pi against key position pj (visible keys only)
__device__ __forceinline__ float wa_score(float dot, const WinAttn &p, float r1, float r2, bool biased, int pi, int pj) {
  float s = dot * p.scale;
  if (p.softcap > 0.f) s = p.softcap * tanhf(s / p.softcap);
  if (biased) s -= r1 * logf(1.0f + r2 * (float)(pi - pj));
  return s;
}

// One warp's scan over the key tiles lo + 32 * (first + k * step), k = 0, 1, ...: running max m, sum l and the weighted sum
// of values acc[i] for dimension lane + 32 i.  q sits in shared memory as fp32.
template <typename T>
__device__ __forceinline__ void wa_scan(const WinAttn &p, const float *q, const T *kc, const T *vc, int lo, int pi, int first, int step,
                                        float r1, float r2, bool biased, int lane, float &m, float &l, float (&acc)[WA_MAX_HD / 32]) {
  constexpr int MAXD = WA_MAX_HD / 32;
  const int hd = p.hd;
  for (int j0 = lo + 32 * first; j0 <= pi; j0 += 32 * step) {
    const int j = j0 + lane;
    const bool vis = j <= pi;
    float s = -INFINITY;
    if (vis) s = wa_score(wa_dot<T>(q, kc + (size_t)j * hd, hd), p, r1, r2, biased, pi, j);
    const float mn = fmaxf(m, warp_max(s));
    const float f = (m == -INFINITY) ? 0.f : expf(m - mn);
    const float e = vis ? expf(s - mn) : 0.f;
    l = l * f + warp_sum(e);
    m = mn;
#pragma unroll
    for (int i = 0; i < MAXD; i++) acc[i] *= f;
    const int cnt = min(32, pi - j0 + 1);
    for (int jj = 0; jj < cnt; jj++) {
      const float pj = __shfl_sync(0xffffffffu, e, jj);
      const T *vr = vc + (size_t)(j0 + jj) * hd;
#pragma unroll
      for (int i = 0; i < MAXD; i++) {
        const int d = lane + 32 * i;
        if (d < hd) acc[i] = fmaf(pj, DT<T>::to_f(vr[d]), acc[i]);
      }
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(128) attn_window_bias_kernel(const WinAttn p) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float qs[4][WA_MAX_HD];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long item = (long)blockIdx.x * 4 + warp;
  if (item >= (long)p.B * p.S * p.heads) return;
  const int h = (int)(item % p.heads);
  const int t = (int)((item / p.heads) % p.S);
  const int b = (int)(item / ((long)p.heads * p.S));
  const int hd = p.hd, G = p.heads / p.n_kv;
  const T *qrow = reinterpret_cast<const T *>(p.qkg) + (size_t)(b * p.S + t) * p.ld;
  const T *kc = reinterpret_cast<const T *>(p.kc) + ((size_t)b * p.n_kv + h / G) * p.cap * hd;
  const T *vc = reinterpret_cast<const T *>(p.vc) + ((size_t)b * p.n_kv + h / G) * p.cap * hd;
  for (int d = lane; d < hd; d += 32) qs[warp][d] = DT<T>::to_f(qrow[h * hd + d]);
  __syncwarp();
  const bool biased = p.r1 != nullptr;
  const float r1 = biased ? DT<T>::to_f(reinterpret_cast<const T *>(p.r1)[h]) : 0.f;
  const float r2 = biased ? DT<T>::to_f(reinterpret_cast<const T *>(p.r2)[h]) : 0.f;
  const int pi = p.pos0 + t;
  const int lo = p.window > 0 ? max(0, pi - p.window + 1) : 0;
  constexpr int MAXD = WA_MAX_HD / 32;
  float acc[MAXD];
#pragma unroll
  for (int i = 0; i < MAXD; i++) acc[i] = 0.f;
  float m = -INFINITY, l = 0.f;
  wa_scan<T>(p, qs[warp], kc, vc, lo, pi, 0, 1, r1, r2, biased, lane, m, l, acc);
  float gate = 1.0f;
  if (p.gate_col >= 0) gate = 1.0f / (1.0f + expf(-DT<T>::to_f(qrow[p.gate_col + h])));
  const float inv = gate / l;
  T *yo = reinterpret_cast<T *>(p.y) + (size_t)(b * p.S + t) * p.ldy + h * hd;
#pragma unroll
  for (int i = 0; i < MAXD; i++) {
    const int d = lane + 32 * i;
    if (d < hd) yo[d] = DT<T>::from_f(acc[i] * inv);
  }
}

// Single-token steps: one CTA per (token, head); its 16 warps take the window's 32-key tiles in turn and merge their
// (m, l, acc) states in shared memory in warp order, so the result does not depend on timing.
constexpr int WA_DEC_WARPS = 16;
template <typename T>
__global__ void __launch_bounds__(WA_DEC_WARPS * 32) attn_window_decode_kernel(const WinAttn p) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float qs[WA_MAX_HD];
  __shared__ float sm_m[WA_DEC_WARPS], sm_l[WA_DEC_WARPS];
  __shared__ float sm_acc[WA_DEC_WARPS][WA_MAX_HD];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int item = blockIdx.x;
  const int h = item % p.heads, t = (item / p.heads) % p.S, b = item / (p.heads * p.S);
  const int hd = p.hd, G = p.heads / p.n_kv;
  const T *qrow = reinterpret_cast<const T *>(p.qkg) + (size_t)(b * p.S + t) * p.ld;
  const T *kc = reinterpret_cast<const T *>(p.kc) + ((size_t)b * p.n_kv + h / G) * p.cap * hd;
  const T *vc = reinterpret_cast<const T *>(p.vc) + ((size_t)b * p.n_kv + h / G) * p.cap * hd;
  for (int d = threadIdx.x; d < hd; d += blockDim.x) qs[d] = DT<T>::to_f(qrow[h * hd + d]);
  __syncthreads();
  const bool biased = p.r1 != nullptr;
  const float r1 = biased ? DT<T>::to_f(reinterpret_cast<const T *>(p.r1)[h]) : 0.f;
  const float r2 = biased ? DT<T>::to_f(reinterpret_cast<const T *>(p.r2)[h]) : 0.f;
  const int pi = p.pos0 + t;
  const int lo = p.window > 0 ? max(0, pi - p.window + 1) : 0;
  constexpr int MAXD = WA_MAX_HD / 32;
  float acc[MAXD];
#pragma unroll
  for (int i = 0; i < MAXD; i++) acc[i] = 0.f;
  float m = -INFINITY, l = 0.f;
  wa_scan<T>(p, qs, kc, vc, lo, pi, warp, WA_DEC_WARPS, r1, r2, biased, lane, m, l, acc);
  if (lane == 0) { sm_m[warp] = m; sm_l[warp] = l; }
#pragma unroll
  for (int i = 0; i < MAXD; i++) {
    const int d = lane + 32 * i;
    if (d < hd) sm_acc[warp][d] = acc[i];
  }
  __syncthreads();
  float mx = -INFINITY;
  for (int w = 0; w < WA_DEC_WARPS; w++) mx = fmaxf(mx, sm_m[w]);
  float lt = 0.f;
  for (int w = 0; w < WA_DEC_WARPS; w++) lt += sm_m[w] == -INFINITY ? 0.f : sm_l[w] * expf(sm_m[w] - mx);
  float gate = 1.0f;
  if (p.gate_col >= 0) gate = 1.0f / (1.0f + expf(-DT<T>::to_f(qrow[p.gate_col + h])));
  const float inv = gate / lt;
  T *yo = reinterpret_cast<T *>(p.y) + (size_t)(b * p.S + t) * p.ldy + h * hd;
  for (int d = threadIdx.x; d < hd; d += blockDim.x) {
    float a = 0.f;
    for (int w = 0; w < WA_DEC_WARPS; w++)
      if (sm_m[w] != -INFINITY) a = fmaf(sm_acc[w][d], expf(sm_m[w] - mx), a);
    yo[d] = DT<T>::from_f(a * inv);
  }
}

// Single-token steps for 16-bit D, head_dim a multiple of 8, values == keys.  Eight lanes share a key: lane r of a group
// holds the 16-byte pieces r, r + 8, ... of the row (NCH of them), so a warp's loads are whole rows, a score costs three
// shuffles, and the registers that fed the dot product also feed the weighted sum (the key is read once).  Every group
// keeps its own running (m, l, acc) over the keys lo + grp, lo + grp + 64, ... with U rows in flight; the groups merge in a
// fixed order — shuffles inside a warp, shared memory across the warps — so the result does not depend on timing.
template <typename T, int NCH>
__global__ void __launch_bounds__(WA_DEC_WARPS * 32) attn_window_decode_vec_kernel(const WinAttn p) {
  pdl_launch_dependents();
  pdl_wait();
  constexpr int NG = WA_DEC_WARPS * 4;  // key groups of a CTA
  constexpr int U = NCH >= 3 ? 2 : 4;   // keys in flight per group
  __shared__ float sm_m[WA_DEC_WARPS], sm_l[WA_DEC_WARPS];
  __shared__ float sm_acc[WA_DEC_WARPS][WA_MAX_HD];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, grp = threadIdx.x >> 3, r = threadIdx.x & 7;
  const int item = blockIdx.x;
  const int h = item % p.heads, t = (item / p.heads) % p.S, b = item / (p.heads * p.S);
  const int hd = p.hd, CH = hd >> 3, G = p.heads / p.n_kv;
  const T *qrow = reinterpret_cast<const T *>(p.qkg) + (size_t)(b * p.S + t) * p.ld;
  const T *kc = reinterpret_cast<const T *>(p.kc) + ((size_t)b * p.n_kv + h / G) * p.cap * hd;
  float q[NCH][8], acc[NCH][8];
#pragma unroll
  for (int c = 0; c < NCH; c++) {
    const int ch = r + 8 * c;
    uint4 v = make_uint4(0u, 0u, 0u, 0u);  // sixteen zero bits are 0.0 in both 16-bit types
    if (ch < CH) v = reinterpret_cast<const uint4 *>(qrow + (size_t)h * hd)[ch];
    unpack8<T>(v, q[c]);
#pragma unroll
    for (int e = 0; e < 8; e++) acc[c][e] = 0.f;
  }
  const bool biased = p.r1 != nullptr;
  const float r1 = biased ? DT<T>::to_f(reinterpret_cast<const T *>(p.r1)[h]) : 0.f;
  const float r2 = biased ? DT<T>::to_f(reinterpret_cast<const T *>(p.r2)[h]) : 0.f;
  const int pi = p.pos0 + t;
  const int lo = p.window > 0 ? max(0, pi - p.window + 1) : 0;
  const float inv_cap2 = p.softcap > 0.f ? 2.0f / p.softcap : 0.f;
  float m = -INFINITY, l = 0.f;
  for (int base = lo; base <= pi; base += NG * U) {  // the trip count is the same for every thread: the shuffles below are whole-warp
    uint4 kr[U][NCH];
#pragma unroll
    for (int u = 0; u < U; u++) {
      const int j = base + u * NG + grp;
#pragma unroll
      for (int c = 0; c < NCH; c++) {
        const int ch = r + 8 * c;
        kr[u][c] = make_uint4(0u, 0u, 0u, 0u);
        if (j <= pi && ch < CH) kr[u][c] = reinterpret_cast<const uint4 *>(kc + (size_t)j * hd)[ch];
      }
    }
#pragma unroll
    for (int u = 0; u < U; u++) {
      const int j = base + u * NG + grp;
      float kf[NCH][8];
      float d = 0.f;
#pragma unroll
      for (int c = 0; c < NCH; c++) {
        unpack8<T>(kr[u][c], kf[c]);
#pragma unroll
        for (int e = 0; e < 8; e++) d = fmaf(q[c][e], kf[c][e], d);
      }
      d += __shfl_xor_sync(0xffffffffu, d, 1);
      d += __shfl_xor_sync(0xffffffffu, d, 2);
      d += __shfl_xor_sync(0xffffffffu, d, 4);
      if (j <= pi) {
        // the modifiers as in the tensor-core kernels below (MUFU-based tanh and ln: |error| ~1e-6 of a score)
        float s = d * p.scale;
        if (p.softcap > 0.f) s = p.softcap * (1.0f - __fdividef(2.0f, __expf(s * inv_cap2) + 1.0f));
        if (biased) s -= r1 * __logf(fmaf(r2, (float)(pi - j), 1.0f));
        if (s > m) {  // a new maximum is rare after the first keys: rescale only then
          const float f = (m == -INFINITY) ? 0.f : __expf(m - s);
          l *= f;
#pragma unroll
          for (int c = 0; c < NCH; c++)
#pragma unroll
            for (int e = 0; e < 8; e++) acc[c][e] *= f;
          m = s;
        }
        const float w = __expf(s - m);
        l += w;
#pragma unroll
        for (int c = 0; c < NCH; c++)
#pragma unroll
          for (int e = 0; e < 8; e++) acc[c][e] = fmaf(w, kf[c][e], acc[c][e]);
      }
    }
  }
  // the four groups of a warp: common maximum, rescale, sum (a + b is the same number on both sides of an exchange)
  float mw = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 8));
  mw = fmaxf(mw, __shfl_xor_sync(0xffffffffu, mw, 16));
  const float sc = (m == -INFINITY) ? 0.f : expf(m - mw);
  l *= sc;
  l += __shfl_xor_sync(0xffffffffu, l, 8);
  l += __shfl_xor_sync(0xffffffffu, l, 16);
#pragma unroll
  for (int c = 0; c < NCH; c++)
#pragma unroll
    for (int e = 0; e < 8; e++) {
      float a = acc[c][e] * sc;
      a += __shfl_xor_sync(0xffffffffu, a, 8);
      a += __shfl_xor_sync(0xffffffffu, a, 16);
      acc[c][e] = a;
    }
  if (lane == 0) { sm_m[warp] = mw; sm_l[warp] = l; }
  if (lane < 8) {
#pragma unroll
    for (int c = 0; c < NCH; c++) {
      const int ch = lane + 8 * c;
      if (ch < CH) {
#pragma unroll
        for (int e = 0; e < 8; e++) sm_acc[warp][ch * 8 + e] = acc[c][e];
      }
    }
  }
  __syncthreads();
  float mx = -INFINITY;
  for (int w = 0; w < WA_DEC_WARPS; w++) mx = fmaxf(mx, sm_m[w]);
  float lt = 0.f;
  for (int w = 0; w < WA_DEC_WARPS; w++) lt += sm_m[w] == -INFINITY ? 0.f : sm_l[w] * expf(sm_m[w] - mx);
  float gate = 1.0f;
  if (p.gate_col >= 0) gate = 1.0f / (1.0f + expf(-DT<T>::to_f(qrow[p.gate_col + h])));
  const float inv = gate / lt;
  T *yo = reinterpret_cast<T *>(p.y) + (size_t)(b * p.S + t) * p.ldy + h * hd;
  for (int d = threadIdx.x; d < hd; d += blockDim.x) {
    float a = 0.f;
    for (int w = 0; w < WA_DEC_WARPS; w++)
      if (sm_m[w] != -INFINITY) a = fmaf(sm_acc[w][d], expf(sm_m[w] - mx), a);
    yo[d] = DT<T>::from_f(a * inv);
  }
}

// ---- prompt portions on the tensor cores (16-bit D, head_dim a multiple of 16) -----------------------------------------------
// Flash-style like attn_prefill_mma_kernel (attn_prefill.cuh): a CTA = 64 query rows of one head (4 warps x 16 rows), key
// tiles of 64 positions through a 2-stage cp.async pipeline, mma.sync m16n8k16 with fp32 accumulation, P = P_hi + P_lo in D.
// Differences: the tile loop starts at the first tile the window reaches; the score gets its soft cap and distance bias
// before the mask; ONE shared-memory tile is both the K operand of Q K^T and — read with ldmatrix.trans — the V operand of
// P V, since the keys double as values; the head gate scales the result.  Rows are padded by 16 bytes (an odd number of
// 16-byte chunks per row keeps ldmatrix conflict-free for every head_dim, also those that are not a power of two).
// tanh and ln use the MUFU-based __expf / __logf: |error| ~1e-6 of the score, two orders below the rounding of q and k to D.
constexpr int WM_BM = 64, WM_BN = 64, WM_THREADS = 128;
template <int HD> __device__ __forceinline__ uint32_t wm_off(int r, int c) { return (uint32_t)(r * (HD * 2 + 16) + (c << 4)); }
template <int HD> constexpr int wm_smem_bytes() { return 3 * WM_BN * (HD * 2 + 16); }

template <typename T, int HD>
__global__ void __launch_bounds__(WM_THREADS, 2) attn_window_mma_kernel(const WinAttn p) {
  constexpr int CH = HD / 8, KS = HD / 16, NT = WM_BN / 8, DTN = HD / 8;
  constexpr int TILE_B = WM_BN * (HD * 2 + 16);
  extern __shared__ __align__(128) unsigned char wm_smem[];
  unsigned char *k_s = wm_smem;               // [2][64][HD + 8]
  unsigned char *q_s = wm_smem + 2 * TILE_B;  // [64][HD + 8]
  pdl_launch_dependents();
  pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int mt = gridDim.x - 1 - blockIdx.x;
  const int h = blockIdx.y, b = blockIdx.z, G = p.heads / p.n_kv;
  const int m0 = mt * WM_BM;
  const T *qkg = reinterpret_cast<const T *>(p.qkg);
  const T *kc = reinterpret_cast<const T *>(p.kc) + ((size_t)b * p.n_kv + h / G) * p.cap * HD;
  const int kv_end = p.pos0 + min(p.S, m0 + WM_BM);                                    // one past the last key this tile's rows see
  const int k_first = p.window > 0 ? max(0, p.pos0 + m0 - p.window + 1) : 0;          // first key its first row sees
  const int j_lo = k_first / WM_BN, n_tiles = (kv_end + WM_BN - 1) / WM_BN;

  auto load_k = [&](int j, int buf) {
    for (int i = threadIdx.x; i < WM_BN * CH; i += WM_THREADS) {
      const int r = i / CH, c = i % CH, key = j * WM_BN + r;
      const bool ok = key < kv_end;
      cp_async16(smem_u32(k_s + buf * TILE_B) + wm_off<HD>(r, c), kc + (size_t)(ok ? key : 0) * HD + c * 8, ok ? 16 : 0);
    }
  };
  for (int i = threadIdx.x; i < WM_BM * CH; i += WM_THREADS) {
    const int r = i / CH, c = i % CH, t = m0 + r;
    const bool ok = t < p.S;
    cp_async16(smem_u32(q_s) + wm_off<HD>(r, c), qkg + (size_t)(b * p.S + (ok ? t : 0)) * p.ld + h * HD + c * 8, ok ? 16 : 0);
  }
  load_k(j_lo, 0);
  cp_async_commit();

  float o[DTN][4];
#pragma unroll
  for (int i = 0; i < DTN; i++) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
  uint32_t qf[KS][4];
  const int g = lane >> 2, c2 = (lane & 3) * 2;
  const int qpos0 = p.pos0 + m0 + warp * 16 + g;
  const int mi = lane >> 3, lr = lane & 7;
  const bool biased = p.r1 != nullptr;
  const float r1 = biased ? DT<T>::to_f(reinterpret_cast<const T *>(p.r1)[h]) : 0.f;
  const float r2 = biased ? DT<T>::to_f(reinterpret_cast<const T *>(p.r2)[h]) : 0.f;
  const float inv_cap2 = p.softcap > 0.f ? 2.0f / p.softcap : 0.f;

  cp_async_wait<0>();
  __syncthreads();
#pragma unroll
  for (int ks = 0; ks < KS; ks++) ldsm_x4(qf[ks], smem_u32(q_s) + wm_off<HD>(warp * 16 + (mi & 1) * 8 + lr, ks * 2 + (mi >> 1)));
  for (int j = j_lo; j < n_tiles; j++) {
    const int buf = (j - j_lo) & 1;
    if (j + 1 < n_tiles) load_k(j + 1, buf ^ 1);
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();
    float s[NT][4];
#pragma unroll
    for (int nt = 0; nt < NT; nt++) s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.f;
    const uint32_t kb_addr = smem_u32(k_s + buf * TILE_B);
#pragma unroll
    for (int ks = 0; ks < KS; ks++) {
#pragma unroll
      for (int np = 0; np < NT / 2; np++) {
        uint32_t kf[4];
        ldsm_x4(kf, kb_addr + wm_off<HD>(np * 16 + (mi >> 1) * 8 + lr, ks * 2 + (mi & 1)));
        FaMma<T>::mma(s[2 * np], qf[ks], kf[0], kf[1]);
        FaMma<T>::mma(s[2 * np + 1], qf[ks], kf[2], kf[3]);
      }
    }
    float mx[2] = {-INFINITY, -INFINITY};
    const float fq0 = (float)(qpos0 - j * WM_BN - c2);   // distance of this thread's first row to its first key of the tile
    const float fwin = p.window > 0 ? (float)p.window : 3.0e38f;
#pragma unroll
    for (int nt = 0; nt < NT; nt++)
#pragma unroll
      for (int e = 0; e < 4; e++) {
        // branch-free (the independent chains interleave); the distance as a float: no I2F on the MUFU pipe
        const float fd = fq0 + (float)((e >> 1) * 8 - nt * 8 - (e & 1));
        float v = s[nt][e] * p.scale;
        if (p.softcap > 0.f) v = p.softcap * (1.0f - __fdividef(2.0f, __expf(v * inv_cap2) + 1.0f));
        if (biased) v -= r1 * __logf(fmaf(r2, fmaxf(fd, 0.f), 1.0f));
        v = (fd >= 0.f && fd < fwin) ? v : -INFINITY;
        s[nt][e] = v;
        mx[e >> 1] = fmaxf(mx[e >> 1], v);
      }
    float fac[2], rs[2] = {0.f, 0.f};
#pragma unroll
    for (int r = 0; r < 2; r++) {
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
      const float mn = fmaxf(m_run[r], mx[r]);
      fac[r] = (m_run[r] == -INFINITY) ? 0.f : __expf(m_run[r] - mn);
      m_run[r] = mn;
    }
#pragma unroll
    for (int nt = 0; nt < NT; nt++)
#pragma unroll
      for (int e = 0; e < 4; e++) {
        const float mn = m_run[e >> 1];
        const float pv = (mn == -INFINITY) ? 0.f : __expf(s[nt][e] - mn);
        s[nt][e] = pv;
        rs[e >> 1] += pv;
      }
#pragma unroll
    for (int r = 0; r < 2; r++) {
      rs[r] += __shfl_xor_sync(0xffffffffu, rs[r], 1);
      rs[r] += __shfl_xor_sync(0xffffffffu, rs[r], 2);
      l_run[r] = l_run[r] * fac[r] + rs[r];
    }
#pragma unroll
    for (int dt = 0; dt < DTN; dt++) {
      o[dt][0] *= fac[0]; o[dt][1] *= fac[0]; o[dt][2] *= fac[1]; o[dt][3] *= fac[1];
    }
#pragma unroll
    for (int kb = 0; kb < WM_BN / 16; kb++) {
      uint32_t ph[4], pl[4];
#pragma unroll
      for (int q = 0; q < 4; q++) {
        const float p0 = s[2 * kb + (q >> 1)][(q & 1) * 2], p1 = s[2 * kb + (q >> 1)][(q & 1) * 2 + 1];
        const float h0 = rnd<T>(p0), h1 = rnd<T>(p1);
        ph[q] = pack2<T>(h0, h1);
        pl[q] = pack2<T>(p0 - h0, p1 - h1);
      }
#pragma unroll
      for (int dp = 0; dp < DTN / 2; dp++) {
        uint32_t vf[4];
        ldsm_x4_trans(vf, kb_addr + wm_off<HD>(kb * 16 + (mi & 1) * 8 + lr, dp * 2 + (mi >> 1)));
        FaMma<T>::mma(o[2 * dp], ph, vf[0], vf[1]);
        FaMma<T>::mma(o[2 * dp], pl, vf[0], vf[1]);
        FaMma<T>::mma(o[2 * dp + 1], ph, vf[2], vf[3]);
        FaMma<T>::mma(o[2 * dp + 1], pl, vf[2], vf[3]);
      }
    }
    __syncthreads();
  }
  cp_async_wait<0>();
#pragma unroll
  for (int r = 0; r < 2; r++) {
    const int t = m0 + warp * 16 + g + r * 8;
    if (t < p.S) {
      const T *qrow = qkg + (size_t)(b * p.S + t) * p.ld;
      float gate = 1.0f;
      if (p.gate_col >= 0) gate = 1.0f / (1.0f + expf(-DT<T>::to_f(qrow[p.gate_col + h])));
      const float inv = gate / l_run[r];
      T *dst = reinterpret_cast<T *>(p.y) + (size_t)(b * p.S + t) * p.ldy + h * HD;
#pragma unroll
      for (int dt = 0; dt < DTN; dt++)
        *reinterpret_cast<uint32_t *>(dst + dt * 8 + c2) = pack2<T>(o[dt][2 * r] * inv, o[dt][2 * r + 1] * inv);
    }
  }
}

}  // namespace cake
