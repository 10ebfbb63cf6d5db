// mixers_window.cu — kernels behind the second half of mixers.cuh: the element-wise squashing norm, RMS norms of column ranges
// (low-rank latents), rotation + unit norm of queries and keys with the cache append, softmax attention over cached keys and
// values with a sliding window, kept first tokens and a sink (per-row form with split keys for short steps, and a tiled
// tensor-core form for portions in 16-bit D), the per-layer token input and the stream / embedding concatenation.
// sm_100a only.  fp32 everywhere the interface says so; D only where a projection, a cache row or a weight is stored.
#include "mixers.cuh"

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <math.h>
#include <algorithm>
#include <stdlib.h>

#include "common.cuh"

namespace cake {
namespace mx {

#define MX_DISPATCH(dtype, ...)                               \
  do {                                                        \
    if ((dtype) == 2) { typedef float T; __VA_ARGS__; }       \
    else if ((dtype) == 1) { typedef __half T; __VA_ARGS__; } \
    else { typedef __nv_bfloat16 T; __VA_ARGS__; }            \
  } while (0)
#define MX_DONE(n)                     \
  do {                                 \
    if (launches) *launches += (n);    \
    return (int)cudaGetLastError();    \
  } while (0)

__device__ __forceinline__ float sigmoid_f(float z) { return 1.0f / (1.0f + expf(-z)); }

// ---------------------------------------------------------------------------------------------- squashing norm
template <typename T>
__global__ void __launch_bounds__(256) tanh_norm_kernel(const TanhNorm p) {
  const int m = blockIdx.x;
  const size_t src = p.rows ? (size_t)p.rows[m] : (size_t)m * p.row_mul + p.row_add;
  const float *y = p.y + src * p.n;
  const float *x = p.x ? p.x + (size_t)m * p.n : nullptr;
  const T *w = reinterpret_cast<const T *>(p.w), *b = reinterpret_cast<const T *>(p.b);
  if ((p.n & 3) == 0) {  // 16-byte loads of the fp32 rows
    for (int i = blockIdx.y * blockDim.x + threadIdx.x; i < p.n / 4; i += gridDim.y * blockDim.x) {
      const float4 v = reinterpret_cast<const float4 *>(y)[i];
      float r[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int e = 0; e < 4; e++) r[e] = fmaf(tanhf(p.alpha * r[e]), DT<T>::to_f(w[4 * i + e]), DT<T>::to_f(b[4 * i + e]));
      if (p.out32) {
        if (x) {
          const float4 xv = reinterpret_cast<const float4 *>(x)[i];
          r[0] += xv.x; r[1] += xv.y; r[2] += xv.z; r[3] += xv.w;
        }
        reinterpret_cast<float4 *>(p.out32 + (size_t)m * p.n)[i] = make_float4(r[0], r[1], r[2], r[3]);
      } else {
        T *o = reinterpret_cast<T *>(p.outD) + (size_t)m * p.n + 4 * i;
#pragma unroll
        for (int e = 0; e < 4; e++) o[e] = DT<T>::from_f(r[e]);
      }
    }
    return;
  }
  for (int i = blockIdx.y * blockDim.x + threadIdx.x; i < p.n; i += gridDim.y * blockDim.x) {
    float r = fmaf(tanhf(p.alpha * y[i]), DT<T>::to_f(w[i]), DT<T>::to_f(b[i]));
    if (p.out32) p.out32[(size_t)m * p.n + i] = x ? x[i] + r : r;
    else reinterpret_cast<T *>(p.outD)[(size_t)m * p.n + i] = DT<T>::from_f(r);
  }
}
int tanh_norm(cudaStream_t st, int dtype, const TanhNorm &p, uint64_t *launches) {
  if (p.M < 1 || p.n < 1 || !p.y || !p.w || !p.b || (!p.out32 && !p.outD)) return (int)cudaErrorInvalidValue;
  const int per = (p.n + 1023) / 1024;  // few rows: several CTAs per row
  MX_DISPATCH(dtype, (tanh_norm_kernel<T><<<dim3(p.M, p.M < 256 ? per : 1), 256, 0, st>>>(p)));
  MX_DONE(1);
}

// ---------------------------------------------------------------------------------------------- RMS norm of a column range
template <typename T>
__global__ void __launch_bounds__(128) rms_cols_kernel(const RmsCols p) {
  __shared__ float red[4];
  const int m = blockIdx.x, b = m / p.S, t = m % p.S;
  const T *in = reinterpret_cast<const T *>(p.in) + (size_t)m * p.ld + p.col;
  const T *w = reinterpret_cast<const T *>(p.w);
  T *out = reinterpret_cast<T *>(p.out) + ((size_t)b * p.out_rows + p.out_row0 + t) * p.ldo;
  float ss = 0.f;
  for (int i = threadIdx.x; i < p.n; i += blockDim.x) {
    const float v = DT<T>::to_f(in[i]);
    ss = fmaf(v, v, ss);
  }
  ss = warp_sum(ss);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
  __syncthreads();
  const float inv = 1.0f / sqrtf((red[0] + red[1] + red[2] + red[3]) / (float)p.n + p.eps);
  for (int i = threadIdx.x; i < p.n; i += blockDim.x) out[i] = DT<T>::from_f(DT<T>::to_f(in[i]) * inv * DT<T>::to_f(w[i]));
}
int rms_cols(cudaStream_t st, int dtype, const RmsCols &p, uint64_t *launches) {
  if (p.M < 1 || p.n < 1 || p.S < 1) return (int)cudaErrorInvalidValue;
  MX_DISPATCH(dtype, (rms_cols_kernel<T><<<p.M, 128, 0, st>>>(p)));
  MX_DONE(1);
}

// ---------------------------------------------------------------------------------------------- rotation, unit norm, append
// entry i of a head whose first `dims` entries are paired (i, i + dims / 2); cs / sn: this position's table row
template <typename T>
__device__ __forceinline__ float rotated_entry(const T *v, int i, int dims, const float *cs, const float *sn) {
  const int half = dims >> 1;
  if (i >= dims) return DT<T>::to_f(v[i]);
  if (i < half) return DT<T>::to_f(v[i]) * cs[i] - DT<T>::to_f(v[i + half]) * sn[i];
  return DT<T>::to_f(v[i]) * cs[i - half] + DT<T>::to_f(v[i - half]) * sn[i - half];
}
template <typename T>
__global__ void __launch_bounds__(256) qk_prep_kernel(const QkPrep p) {
  const int m = blockIdx.x, b = m / p.S, t = m % p.S, pos = p.pos0 + t;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  const T *row = reinterpret_cast<const T *>(p.proj) + (size_t)m * p.ld;
  const int dims = p.cos_t ? p.rope_dims : 0, half = dims >> 1;
  const float *cs = p.cos_t ? p.cos_t + (size_t)pos * half : nullptr, *sn = p.sin_t ? p.sin_t + (size_t)pos * half : nullptr;
  for (int hv = warp; hv < p.heads + p.kv_heads; hv += nw) {
    const bool is_q = hv < p.heads;
    const int g = hv - p.heads;
    const T *v = is_q ? row + p.q_col + (size_t)hv * p.dim : row + p.k_col + (size_t)g * p.dim;
    T *o = is_q ? reinterpret_cast<T *>(p.q_out) + ((size_t)m * p.heads + hv) * p.dim
                : reinterpret_cast<T *>(p.kc) + (((size_t)b * p.kv_heads + g) * p.cap + pos) * p.dim;
    float inv = 1.f;
    if (p.unit_norm) {
      float ss = 0.f;
      for (int i = lane; i < p.dim; i += 32) {
        const float r = rotated_entry<T>(v, i, dims, cs, sn);
        ss = fmaf(r, r, ss);
      }
      ss = warp_sum(ss);
      inv = 1.0f / sqrtf(ss / (float)p.dim + p.eps);
    }
    for (int i = lane; i < p.dim; i += 32) o[i] = DT<T>::from_f(rotated_entry<T>(v, i, dims, cs, sn) * inv);
  }
  for (int i = threadIdx.x; i < p.kv_heads * p.vdim; i += blockDim.x) {
    const int g = i / p.vdim, e = i % p.vdim;
    reinterpret_cast<T *>(p.vc)[(((size_t)b * p.kv_heads + g) * p.cap + pos) * p.vdim + e] = row[p.v_col + i];
  }
}
// The same for 16-bit D with head size 32 E (E = 2, 4, 8): a lane owns E adjacent entries of a head, so a head is one vector load
// (two in the rotated part: the entries and their partners half the rotated width away), one vector load of cos and of sin, one
// vector store.  The rotated half-width is a multiple of E, columns and strides multiples of 8.
template <int E> __device__ __forceinline__ void load_words(const void *src, uint32_t (&w)[E / 2]) {
  if (E == 2) w[0] = *reinterpret_cast<const uint32_t *>(src);
  else if (E == 4) { const uint2 t = *reinterpret_cast<const uint2 *>(src); w[0] = t.x; w[1] = t.y; }
  else { const uint4 t = *reinterpret_cast<const uint4 *>(src); w[0] = t.x; w[1] = t.y; w[2] = t.z; w[3] = t.w; }
}
template <int E> __device__ __forceinline__ void load_floats(const float *src, float (&f)[E]) {
  if (E == 2) { const float2 t = *reinterpret_cast<const float2 *>(src); f[0] = t.x; f[1] = t.y; }
  else {
#pragma unroll
    for (int q = 0; q < E / 4; q++) {
      const float4 t = reinterpret_cast<const float4 *>(src)[q];
      f[4 * q] = t.x; f[4 * q + 1] = t.y; f[4 * q + 2] = t.z; f[4 * q + 3] = t.w;
    }
  }
}
template <typename T, int E>
__global__ void __launch_bounds__(256) qk_prep_vec_kernel(const QkPrep p) {
  const int m = blockIdx.x, b = m / p.S, t = m % p.S, pos = p.pos0 + t;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  const T *row = reinterpret_cast<const T *>(p.proj) + (size_t)m * p.ld;
  const int dims = p.cos_t ? p.rope_dims : 0, half = dims >> 1, i0 = lane * E;
  const float *cs = p.cos_t ? p.cos_t + (size_t)pos * half : nullptr, *sn = p.sin_t ? p.sin_t + (size_t)pos * half : nullptr;
  for (int hv = warp; hv < p.heads + p.kv_heads; hv += nw) {
    const bool is_q = hv < p.heads;
    const int g = hv - p.heads;
    const T *v = is_q ? row + p.q_col + (size_t)hv * p.dim : row + p.k_col + (size_t)g * p.dim;
    T *o = is_q ? reinterpret_cast<T *>(p.q_out) + ((size_t)m * p.heads + hv) * p.dim
                : reinterpret_cast<T *>(p.kc) + (((size_t)b * p.kv_heads + g) * p.cap + pos) * p.dim;
    uint32_t wa[E / 2];
    load_words<E>(v + i0, wa);
    float r[E];
#pragma unroll
    for (int q = 0; q < E / 2; q++) {
      const float2 f = DT<T>::unpack2(wa[q]);
      r[2 * q] = f.x;
      r[2 * q + 1] = f.y;
    }
    if (i0 < dims) {
      const bool lo = i0 < half;
      uint32_t wb[E / 2];
      load_words<E>(v + (lo ? i0 + half : i0 - half), wb);
      float c[E], sfac[E];
      load_floats<E>(cs + (lo ? i0 : i0 - half), c);
      load_floats<E>(sn + (lo ? i0 : i0 - half), sfac);
#pragma unroll
      for (int q = 0; q < E / 2; q++) {
        const float2 f = DT<T>::unpack2(wb[q]);
        r[2 * q] = lo ? r[2 * q] * c[2 * q] - f.x * sfac[2 * q] : r[2 * q] * c[2 * q] + f.x * sfac[2 * q];
        r[2 * q + 1] = lo ? r[2 * q + 1] * c[2 * q + 1] - f.y * sfac[2 * q + 1] : r[2 * q + 1] * c[2 * q + 1] + f.y * sfac[2 * q + 1];
      }
    }
    float inv = 1.f;
    if (p.unit_norm) {
      float ss = 0.f;
#pragma unroll
      for (int q = 0; q < E; q++) ss = fmaf(r[q], r[q], ss);
      ss = warp_sum(ss);
      inv = 1.0f / sqrtf(ss / (float)p.dim + p.eps);
    }
    uint32_t wo[E / 2];
#pragma unroll
    for (int q = 0; q < E / 2; q++) wo[q] = pack2x<T>(r[2 * q] * inv, r[2 * q + 1] * inv);
    if (E == 2) *reinterpret_cast<uint32_t *>(o + i0) = wo[0];
    else if (E == 4) *reinterpret_cast<uint2 *>(o + i0) = make_uint2(wo[0], wo[1]);
    else *reinterpret_cast<uint4 *>(o + i0) = make_uint4(wo[0], wo[E / 2 > 1 ? 1 : 0], wo[E / 2 > 2 ? 2 : 0], wo[E / 2 > 3 ? 3 : 0]);
  }
  const int vrow = p.kv_heads * p.vdim;  // values: 16-byte pieces (vdim, v_col multiples of 8)
  for (int i = threadIdx.x * 8; i < vrow; i += blockDim.x * 8) {
    const int g = i / p.vdim, e = i % p.vdim;
    *reinterpret_cast<uint4 *>(reinterpret_cast<T *>(p.vc) + (((size_t)b * p.kv_heads + g) * p.cap + pos) * p.vdim + e) =
        *reinterpret_cast<const uint4 *>(row + p.v_col + i);
  }
}
template <typename T> static bool qk_prep_vec(cudaStream_t st, const QkPrep &p) {
  const int E = p.dim / 32, half = p.cos_t ? p.rope_dims / 2 : 0;
  const bool ok = p.dim % 32 == 0 && (E == 2 || E == 4 || E == 8) && half % E == 0 && p.vdim % 8 == 0 && p.ld % 8 == 0 && p.q_col % 8 == 0 &&
                  p.k_col % 8 == 0 && p.v_col % 8 == 0 &&
                  (((uintptr_t)p.proj | (uintptr_t)p.q_out | (uintptr_t)p.kc | (uintptr_t)p.vc | (uintptr_t)p.cos_t | (uintptr_t)p.sin_t) & 15) == 0 &&
                  (half * sizeof(float)) % 16 == 0;
  if (!ok) return false;
  const unsigned nt = (p.heads + p.kv_heads) > 4 ? 256 : 128;
  if (E == 2) qk_prep_vec_kernel<T, 2><<<p.B * p.S, nt, 0, st>>>(p);
  else if (E == 4) qk_prep_vec_kernel<T, 4><<<p.B * p.S, nt, 0, st>>>(p);
  else qk_prep_vec_kernel<T, 8><<<p.B * p.S, nt, 0, st>>>(p);
  return true;
}
template <> bool qk_prep_vec<float>(cudaStream_t, const QkPrep &) { return false; }
int qk_prep(cudaStream_t st, int dtype, const QkPrep &p, uint64_t *launches) {
  if (p.B < 1 || p.S < 1 || p.heads < 1 || p.kv_heads < 1 || (p.cos_t && (p.rope_dims & 1 || p.rope_dims > p.dim))) return (int)cudaErrorInvalidValue;
  bool done = false;
  MX_DISPATCH(dtype, (done = qk_prep_vec<T>(st, p)));
  if (done) MX_DONE(1);
  MX_DISPATCH(dtype, (qk_prep_kernel<T><<<p.B * p.S, (p.heads + p.kv_heads) > 4 ? 256 : 128, 0, st>>>(p)));
  MX_DONE(1);
}

// ---------------------------------------------------------------------------------------------- window attention, per row
// CTA (row-head, split): the visible keys are the kept first tokens that have left the window, then the window; the CTA's
// four warps walk its share four keys at a time each (lanes split the columns of a key and of a value row), their running
// softmax states are merged in shared memory.  Without splits the CTA adds the sink, normalises, gates and writes the output;
// with splits it leaves (max, sum, weighted values) for the merge kernel.
template <typename T, int NR>
__global__ void __launch_bounds__(128) window_attn_kernel(const WindowAttn p) {
  __shared__ float sm_m[4], sm_l[4];
  extern __shared__ float sm_acc[];  // [4][vdim]
  const int mh = blockIdx.x, split = blockIdx.y, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m = mh / p.heads, h = mh % p.heads, b = m / p.S, t = m % p.S, pos = p.pos0 + t;
  const int g = h / (p.heads / p.kv_heads);
  const int lo = p.window > 0 ? max(0, pos - p.window + 1) : 0;
  const int nA = min(p.keep_first, lo), total = nA + pos - lo + 1;
  const int nsplit = p.nsplit > 1 ? p.nsplit : 1;
  const int per = nsplit > 1 ? ((total + nsplit - 1) / nsplit + 15) / 16 * 16 : total;
  const int k0 = split * per, k1 = min(total, k0 + per);
  const T *q = reinterpret_cast<const T *>(p.q) + (size_t)m * p.ldq + (size_t)h * p.dim;
  const T *kc = reinterpret_cast<const T *>(p.kc) + ((size_t)b * p.kv_heads + g) * p.cap * p.dim;
  const T *vc = reinterpret_cast<const T *>(p.vc) + ((size_t)b * p.kv_heads + g) * p.cap * p.vdim;
  const bool shared_rows = p.kc == p.vc && p.dim == p.vdim;  // a key row is also the value row
  float qv[NR], acc[NR];
#pragma unroll
  for (int i = 0; i < NR; i++) {
    const int c = lane + 32 * i;
    qv[i] = c < p.dim ? DT<T>::to_f(q[c]) * p.scale : 0.f;
    acc[i] = 0.f;
  }
  float mx = -INFINITY, l = 0.f;
  for (int jj = k0 + 4 * warp; jj < k1; jj += 16) {
    float vv[4][NR], s[4];
#pragma unroll
    for (int u = 0; u < 4; u++) {
      const int ju = jj + u < k1 ? jj + u : jj;
      const int j = ju < nA ? ju : lo + ju - nA;
      const T *krow = kc + (size_t)j * p.dim;
      float part = 0.f;
      if (shared_rows) {
#pragma unroll
        for (int i = 0; i < NR; i++) {
          const int c = lane + 32 * i;
          vv[u][i] = c < p.dim ? DT<T>::to_f(krow[c]) : 0.f;
          part = fmaf(qv[i], vv[u][i], part);
        }
      } else {
        const T *vrow = vc + (size_t)j * p.vdim;
#pragma unroll
        for (int i = 0; i < NR; i++) {
          const int c = lane + 32 * i;
          part = fmaf(qv[i], c < p.dim ? DT<T>::to_f(krow[c]) : 0.f, part);
          vv[u][i] = c < p.vdim ? DT<T>::to_f(vrow[c]) : 0.f;
        }
      }
      s[u] = part;
    }
#pragma unroll
    for (int u = 0; u < 4; u++) {
      s[u] = warp_sum(s[u]);
      if (jj + u >= k1) s[u] = -INFINITY;
    }
    const float mn = fmaxf(fmaxf(mx, fmaxf(s[0], s[1])), fmaxf(s[2], s[3]));
    const float corr = expf(mx - mn);  // first round: exp(-inf) = 0
    float pr[4];
#pragma unroll
    for (int u = 0; u < 4; u++) pr[u] = expf(s[u] - mn);
    l = l * corr + ((pr[0] + pr[1]) + (pr[2] + pr[3]));
#pragma unroll
    for (int i = 0; i < NR; i++) {
      float a = acc[i] * corr;
#pragma unroll
      for (int u = 0; u < 4; u++) a = fmaf(pr[u], vv[u][i], a);
      acc[i] = a;
    }
    mx = mn;
  }
  if (lane == 0) { sm_m[warp] = mx; sm_l[warp] = l; }
#pragma unroll
  for (int i = 0; i < NR; i++) {
    const int c = lane + 32 * i;
    if (c < p.vdim) sm_acc[warp * p.vdim + c] = acc[i];
  }
  __syncthreads();
  float M4 = fmaxf(fmaxf(sm_m[0], sm_m[1]), fmaxf(sm_m[2], sm_m[3]));
  float f[4], L = 0.f;
  if (nsplit > 1) {
#pragma unroll
    for (int w = 0; w < 4; w++) {
      f[w] = sm_m[w] == -INFINITY ? 0.f : expf(sm_m[w] - M4);
      L = fmaf(sm_l[w], f[w], L);
    }
    float *out = p.part + ((size_t)mh * nsplit + split) * (p.vdim + 2);
    if (threadIdx.x == 0) { out[0] = M4; out[1] = L; }
    for (int c = threadIdx.x; c < p.vdim; c += blockDim.x)
      out[2 + c] = (sm_acc[c] * f[0] + sm_acc[p.vdim + c] * f[1]) + (sm_acc[2 * p.vdim + c] * f[2] + sm_acc[3 * p.vdim + c] * f[3]);
    return;
  }
  float sink_term = 0.f;
  if (p.sink) {
    const float sk = DT<T>::to_f(reinterpret_cast<const T *>(p.sink)[h]);
    M4 = fmaxf(M4, sk);
    sink_term = expf(sk - M4);
  }
#pragma unroll
  for (int w = 0; w < 4; w++) {
    f[w] = sm_m[w] == -INFINITY ? 0.f : expf(sm_m[w] - M4);
    L = fmaf(sm_l[w], f[w], L);
  }
  const float il = 1.0f / (L + sink_term);
  const T *gate = reinterpret_cast<const T *>(p.gate);
  const float gh = gate && p.gate_per_head ? sigmoid_f(DT<T>::to_f(gate[(size_t)m * p.ldg + h])) : 1.f;
  T *out = reinterpret_cast<T *>(p.out) + (size_t)m * p.ldo + (size_t)h * p.vdim;
  for (int c = threadIdx.x; c < p.vdim; c += blockDim.x) {
    float o = ((sm_acc[c] * f[0] + sm_acc[p.vdim + c] * f[1]) + (sm_acc[2 * p.vdim + c] * f[2] + sm_acc[3 * p.vdim + c] * f[3])) * il;
    if (gate) o *= p.gate_per_head ? gh : sigmoid_f(DT<T>::to_f(gate[(size_t)m * p.ldg + (size_t)h * p.vdim + c]));
    out[c] = DT<T>::from_f(o);
  }
}
template <typename T>
__global__ void __launch_bounds__(128) window_attn_merge_kernel(const WindowAttn p) {
  const int mh = blockIdx.x, m = mh / p.heads, h = mh % p.heads, stride = p.vdim + 2;
  const float *part = p.part + (size_t)mh * p.nsplit * stride;
  float M = p.sink ? DT<T>::to_f(reinterpret_cast<const T *>(p.sink)[h]) : -INFINITY;
  float L = p.sink ? 1.f : 0.f;  // the sink's term relative to its own logit; rescaled below
  const float sk = M;
  for (int s = 0; s < p.nsplit; s++) M = fmaxf(M, part[(size_t)s * stride]);
  L = p.sink ? expf(sk - M) : 0.f;
  for (int s = 0; s < p.nsplit; s++) {
    const float ms = part[(size_t)s * stride];
    if (ms != -INFINITY) L = fmaf(part[(size_t)s * stride + 1], expf(ms - M), L);
  }
  const T *gate = reinterpret_cast<const T *>(p.gate);
  const float gh = gate && p.gate_per_head ? sigmoid_f(DT<T>::to_f(gate[(size_t)m * p.ldg + h])) : 1.f;
  T *out = reinterpret_cast<T *>(p.out) + (size_t)m * p.ldo + (size_t)h * p.vdim;
  for (int c = threadIdx.x; c < p.vdim; c += blockDim.x) {
    float a = 0.f;
    for (int s = 0; s < p.nsplit; s++) {
      const float ms = part[(size_t)s * stride];
      if (ms != -INFINITY) a = fmaf(part[(size_t)s * stride + 2 + c], expf(ms - M), a);
    }
    float o = a / L;
    if (gate) o *= p.gate_per_head ? gh : sigmoid_f(DT<T>::to_f(gate[(size_t)m * p.ldg + (size_t)h * p.vdim + c]));
    out[c] = DT<T>::from_f(o);
  }
}
int window_attention(cudaStream_t st, int dtype, const WindowAttn &p, uint64_t *launches) {
  const int D = p.dim > p.vdim ? p.dim : p.vdim;
  if (D > 32 * 24 || p.heads < 1 || p.kv_heads < 1 || p.heads % p.kv_heads || p.window < 0 || p.keep_first < 0) return (int)cudaErrorInvalidValue;
  const bool split = p.part && p.nsplit > 1;
  const dim3 grid((unsigned)(p.B * p.S * p.heads), (unsigned)(split ? p.nsplit : 1));
  const size_t smem = (size_t)4 * p.vdim * sizeof(float);
  MX_DISPATCH(dtype, {
    if (D <= 32 * 2) window_attn_kernel<T, 2><<<grid, 128, smem, st>>>(p);
    else if (D <= 32 * 4) window_attn_kernel<T, 4><<<grid, 128, smem, st>>>(p);
    else if (D <= 32 * 8) window_attn_kernel<T, 8><<<grid, 128, smem, st>>>(p);
    else if (D <= 32 * 16) window_attn_kernel<T, 16><<<grid, 128, smem, st>>>(p);
    else window_attn_kernel<T, 24><<<grid, 128, smem, st>>>(p);
    if (split) window_attn_merge_kernel<T><<<grid.x, 128, 0, st>>>(p);
  });
  MX_DONE(split ? 2 : 1);
}

// ---------------------------------------------------------------------------------------------- window attention, tiled
// A CTA of four warps owns 64 consecutive rows of one (batch row, head); every warp 16 of them.  Keys come in tiles of 64: first
// the kept first tokens that lie before the window of the block's first row, then the window up to the block's last row; the
// visibility rule is applied per score, so a tile may straddle any edge.  Scores are 16 x 8 x 16 tensor-core products of the
// staged q and key tiles with fp32 accumulators; the running softmax is fp32 per row (a quad of lanes shares a row); the weights
// enter the second product as w_hi + w_lo in D (about 16 mantissa bits), the values through transposing shared-memory loads.
// Head sizes are padded to the template's with zero columns in shared memory.
constexpr int WT_ROWS = 64, WT_KEYS = 64;
template <typename T> __device__ __forceinline__ void mma16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1);
template <> __device__ __forceinline__ void mma16816<__nv_bfloat16>(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
template <> __device__ __forceinline__ void mma16816<__half>(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// rows [r0, r0 + 64) of a [*, width] matrix with row stride ld into a tile with row stride LDS; rows >= n_rows and columns >= width
// are zeros (width is a multiple of 8: 16-byte pieces)
template <typename T, int LDS, int COLS>
__device__ __forceinline__ void stage_tile(T *dst, const T *src, long ld, int n_rows, int width) {
  constexpr int PIECES = COLS / 8;
  for (int i = threadIdx.x; i < 64 * PIECES; i += blockDim.x) {
    const int r = i / PIECES, c = (i % PIECES) * 8;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (r < n_rows && c < width) v = *reinterpret_cast<const uint4 *>(src + (long)r * ld + c);
    *reinterpret_cast<uint4 *>(dst + r * LDS + c) = v;
  }
}
template <typename T, int HD>
__global__ void __launch_bounds__(128) window_attn_tiled_kernel(const WindowAttn p) {
  constexpr int LDS = HD + 8, KS = HD / 16, NV = HD / 8;
  extern __shared__ __align__(16) unsigned char wt_smem[];
  T *qs = reinterpret_cast<T *>(wt_smem), *ks = qs + 64 * LDS, *vs = ks + 64 * LDS;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, gid = lane >> 2, qd = lane & 3;
  const int r0 = blockIdx.x * WT_ROWS, h = blockIdx.y, b = blockIdx.z, g = h / (p.heads / p.kv_heads);
  const int n_rows = min(WT_ROWS, p.S - r0), p0 = p.pos0 + r0, p1 = p0 + n_rows - 1;
  const T *q = reinterpret_cast<const T *>(p.q) + ((size_t)b * p.S + r0) * p.ldq + (size_t)h * p.dim;
  const T *kc = reinterpret_cast<const T *>(p.kc) + ((size_t)b * p.kv_heads + g) * p.cap * p.dim;
  const T *vc = reinterpret_cast<const T *>(p.vc) + ((size_t)b * p.kv_heads + g) * p.cap * p.vdim;
  stage_tile<T, LDS, HD>(qs, q, p.ldq, n_rows, p.dim);
  __syncthreads();
  uint32_t qf[KS][4];
#pragma unroll
  for (int kk = 0; kk < KS; kk++) {
    const T *base = qs + (warp * 16 + gid) * LDS + kk * 16 + 2 * qd;
    qf[kk][0] = *reinterpret_cast<const uint32_t *>(base);
    qf[kk][1] = *reinterpret_cast<const uint32_t *>(base + 8 * LDS);
    qf[kk][2] = *reinterpret_cast<const uint32_t *>(base + 8);
    qf[kk][3] = *reinterpret_cast<const uint32_t *>(base + 8 * LDS + 8);
  }
  float o[NV][4];
#pragma unroll
  for (int n = 0; n < NV; n++) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;
  float mrow[2] = {-INFINITY, -INFINITY}, lrow[2] = {0.f, 0.f};
  const int row_pos[2] = {p0 + warp * 16 + gid, p0 + warp * 16 + gid + 8};
  const int lo = p.window > 0 ? max(0, p0 - p.window + 1) : 0;
  const int nA = min(p.keep_first, lo);
  const int tilesA = (nA + WT_KEYS - 1) / WT_KEYS, tilesB = (p1 - lo + 1 + WT_KEYS - 1) / WT_KEYS;
  for (int tl = 0; tl < tilesA + tilesB; tl++) {
    const int j0 = tl < tilesA ? tl * WT_KEYS : lo + (tl - tilesA) * WT_KEYS;
    const int jend = tl < tilesA ? nA : p1 + 1;            // keys of this tile: [j0, min(j0 + 64, jend))
    const int nk = min(WT_KEYS, jend - j0);
    __syncthreads();                                        // the previous tile has been consumed
    stage_tile<T, LDS, HD>(ks, kc + (size_t)j0 * p.dim, p.dim, nk, p.dim);
    stage_tile<T, LDS, HD>(vs, vc + (size_t)j0 * p.vdim, p.vdim, nk, p.vdim);
    __syncthreads();
    float sc[8][4];
#pragma unroll
    for (int n = 0; n < 8; n++) {
      sc[n][0] = sc[n][1] = sc[n][2] = sc[n][3] = 0.f;
#pragma unroll
      for (int kk = 0; kk < KS; kk++) {
        const T *kb = ks + (n * 8 + gid) * LDS + kk * 16 + 2 * qd;
        mma16816<T>(sc[n], qf[kk], *reinterpret_cast<const uint32_t *>(kb), *reinterpret_cast<const uint32_t *>(kb + 8));
      }
    }
    // visibility, scale, running maximum
    float mnew[2] = {mrow[0], mrow[1]};
#pragma unroll
    for (int n = 0; n < 8; n++)
#pragma unroll
      for (int e = 0; e < 4; e++) {
        const int j = j0 + n * 8 + 2 * qd + (e & 1), i = row_pos[e >> 1];
        const bool vis = j < jend && j <= i && (p.window == 0 || i - j < p.window || j < p.keep_first);
        sc[n][e] = vis ? sc[n][e] * p.scale : -INFINITY;
        mnew[e >> 1] = fmaxf(mnew[e >> 1], sc[n][e]);
      }
    float corr[2];
#pragma unroll
    for (int r = 0; r < 2; r++) {
      mnew[r] = fmaxf(mnew[r], __shfl_xor_sync(0xffffffffu, mnew[r], 1));
      mnew[r] = fmaxf(mnew[r], __shfl_xor_sync(0xffffffffu, mnew[r], 2));
      corr[r] = mnew[r] == -INFINITY ? 1.f : expf(mrow[r] - mnew[r]);
      mrow[r] = mnew[r];
      lrow[r] *= corr[r];
    }
#pragma unroll
    for (int n = 0; n < NV; n++) {
      o[n][0] *= corr[0]; o[n][1] *= corr[0]; o[n][2] *= corr[1]; o[n][3] *= corr[1];
    }
    // weights as w_hi + w_lo in D, in the first operand's layout: score tiles 2 kk and 2 kk + 1 form the k-step kk
    uint32_t wh[4][4], wl[4][4];
#pragma unroll
    for (int n = 0; n < 8; n++) {
      float w[4];
#pragma unroll
      for (int e = 0; e < 4; e++) {
        w[e] = mrow[e >> 1] == -INFINITY ? 0.f : expf(sc[n][e] - mrow[e >> 1]);
        lrow[e >> 1] += w[e];
      }
      const int kk = n >> 1, off = (n & 1) * 2;
      wh[kk][off] = pack2x<T>(w[0], w[1]);
      wh[kk][off + 1] = pack2x<T>(w[2], w[3]);
      wl[kk][off] = pack2x<T>(w[0] - rnd<T>(w[0]), w[1] - rnd<T>(w[1]));
      wl[kk][off + 1] = pack2x<T>(w[2] - rnd<T>(w[2]), w[3] - rnd<T>(w[3]));
    }
#pragma unroll
    for (int kk = 0; kk < 4; kk++)
#pragma unroll
      for (int n = 0; n < NV; n++) {
        uint32_t b0, b1;
        const T *vrow = vs + (kk * 16 + (lane & 15)) * LDS + n * 8;
        const uint32_t addr = (uint32_t)__cvta_generic_to_shared(vrow);
        asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0,%1}, [%2];\n" : "=r"(b0), "=r"(b1) : "r"(addr));
        mma16816<T>(o[n], wh[kk], b0, b1);
        mma16816<T>(o[n], wl[kk], b0, b1);
      }
  }
  // the sink joins the denominator; normalise, gate, store
  const T *gate = reinterpret_cast<const T *>(p.gate);
#pragma unroll
  for (int r = 0; r < 2; r++) {
    float l = lrow[r];
    l += __shfl_xor_sync(0xffffffffu, l, 1);
    l += __shfl_xor_sync(0xffffffffu, l, 2);
    float m = mrow[r], f = 1.f;
    if (p.sink) {
      const float sk = DT<T>::to_f(reinterpret_cast<const T *>(p.sink)[h]);
      const float mt = fmaxf(m, sk);
      f = m == -INFINITY ? 0.f : expf(m - mt);
      l = l * f + expf(sk - mt);
    }
    const int row = warp * 16 + gid + 8 * r;
    if (row >= n_rows) continue;
    const float il = f / l;
    const size_t mrow_idx = (size_t)b * p.S + r0 + row;
    const float gh = gate && p.gate_per_head ? sigmoid_f(DT<T>::to_f(gate[mrow_idx * p.ldg + h])) : 1.f;
    T *out = reinterpret_cast<T *>(p.out) + mrow_idx * p.ldo + (size_t)h * p.vdim;
#pragma unroll
    for (int n = 0; n < NV; n++) {
      const int c = n * 8 + 2 * qd;
      if (c >= p.vdim) continue;
      float v0 = o[n][2 * r] * il, v1 = o[n][2 * r + 1] * il;
      if (gate) {
        v0 *= p.gate_per_head ? gh : sigmoid_f(DT<T>::to_f(gate[mrow_idx * p.ldg + (size_t)h * p.vdim + c]));
        v1 *= p.gate_per_head ? gh : sigmoid_f(DT<T>::to_f(gate[mrow_idx * p.ldg + (size_t)h * p.vdim + c + 1]));
      }
      *reinterpret_cast<uint32_t *>(out + c) = pack2x<T>(v0, v1);
    }
  }
}
template <> __global__ void window_attn_tiled_kernel<float, 32>(const WindowAttn) {}
template <> __global__ void window_attn_tiled_kernel<float, 64>(const WindowAttn) {}
template <> __global__ void window_attn_tiled_kernel<float, 128>(const WindowAttn) {}

bool window_attention_tiled_ok(int dtype, const WindowAttn &p) {
  static const bool off = []() {
    const char *e = getenv("CAKE_B200_NO_TC"), *f = getenv("CAKE_B200_NO_TILED_ATTN");
    return (e && e[0] == '1') || (f && f[0] == '1');
  }();
  const int D = p.dim > p.vdim ? p.dim : p.vdim;
  return !off && dtype != 2 && p.S >= 16 && D <= 128 && p.dim % 8 == 0 && p.vdim % 8 == 0 && p.ldq % 8 == 0 && p.ldo % 2 == 0 && p.heads % p.kv_heads == 0 &&
         ((uintptr_t)p.q & 15) == 0 && ((uintptr_t)p.kc & 15) == 0 && ((uintptr_t)p.vc & 15) == 0 && ((uintptr_t)p.out & 3) == 0;
}
template <typename T, int HD> static cudaError_t launch_window_tiled(cudaStream_t st, const WindowAttn &p) {
  const size_t smem = (size_t)3 * 64 * (HD + 8) * sizeof(T);
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(window_attn_tiled_kernel<T, HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
  }
  window_attn_tiled_kernel<T, HD><<<dim3((p.S + WT_ROWS - 1) / WT_ROWS, p.heads, p.B), 128, smem, st>>>(p);
  return cudaSuccess;
}
int window_attention_tiled(cudaStream_t st, int dtype, const WindowAttn &p, uint64_t *launches) {
  if (!window_attention_tiled_ok(dtype, p)) return (int)cudaErrorInvalidValue;
  const int D = p.dim > p.vdim ? p.dim : p.vdim;
  cudaError_t e = cudaSuccess;
  if (dtype == 1) e = D <= 32 ? launch_window_tiled<__half, 32>(st, p) : D <= 64 ? launch_window_tiled<__half, 64>(st, p) : launch_window_tiled<__half, 128>(st, p);
  else e = D <= 32 ? launch_window_tiled<__nv_bfloat16, 32>(st, p) : D <= 64 ? launch_window_tiled<__nv_bfloat16, 64>(st, p) : launch_window_tiled<__nv_bfloat16, 128>(st, p);
  if (e != cudaSuccess) return (int)e;
  MX_DONE(1);
}

// ---------------------------------------------------------------------------------------------- per-layer token input
template <typename T>
__global__ void __launch_bounds__(256) rows_to_d_kernel(const float *__restrict__ x, T *__restrict__ out, size_t n) {
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  const size_t n4 = ((((uintptr_t)x | (uintptr_t)out) & 15) == 0) ? n / 4 : 0;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += stride) {
    const float4 v = reinterpret_cast<const float4 *>(x)[i];
    T *o = out + 4 * i;
    o[0] = DT<T>::from_f(v.x); o[1] = DT<T>::from_f(v.y); o[2] = DT<T>::from_f(v.z); o[3] = DT<T>::from_f(v.w);
  }
  for (size_t i = 4 * n4 + (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) out[i] = DT<T>::from_f(x[i]);
}
int rows_to_d(cudaStream_t st, int dtype, const float *x, void *out, size_t n, uint64_t *launches) {
  if (!x || !out || n < 1) return (int)cudaErrorInvalidValue;
  const unsigned grid = (unsigned)std::min<size_t>((n / 4 + 255) / 256 + 1, 148 * 16);
  MX_DISPATCH(dtype, (rows_to_d_kernel<T><<<grid, 256, 0, st>>>(x, reinterpret_cast<T *>(out), n)));
  MX_DONE(1);
}
template <typename T>
__global__ void __launch_bounds__(256) side_gate_kernel(const SideGate p) {
  const size_t total = (size_t)p.M * p.dim;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const size_t m = i / p.dim;
    const int j = (int)(i % p.dim);
    T *g = reinterpret_cast<T *>(p.g) + m * p.ld + j;
    const float d = DT<T>::to_f(*g);
    const float e = DT<T>::to_f(reinterpret_cast<const T *>(p.table)[(size_t)p.ids[m] * p.table_ld + p.col + j]);
    *g = DT<T>::from_f(0.5f * d * (1.0f + tanhf(0.7978845608028654f * (d + 0.044715f * d * d * d))) * e);
  }
}
int side_gate(cudaStream_t st, int dtype, const SideGate &p, uint64_t *launches) {
  if (p.M < 1 || p.dim < 1 || !p.g || !p.ids || !p.table) return (int)cudaErrorInvalidValue;
  const unsigned grid = (unsigned)std::min<size_t>(((size_t)p.M * p.dim + 255) / 256, 148 * 16);
  MX_DISPATCH(dtype, (side_gate_kernel<T><<<grid, 256, 0, st>>>(p)));
  MX_DONE(1);
}

// ---------------------------------------------------------------------------------------------- [x | x0] in D
template <typename T>
__global__ void __launch_bounds__(256) concat_rows_kernel(const float *__restrict__ x, const float *__restrict__ x0, T *__restrict__ out, int W) {
  const size_t m = blockIdx.x;
  for (int i = threadIdx.x; i < W; i += blockDim.x) {
    out[m * 2 * W + i] = DT<T>::from_f(x[m * W + i]);
    out[m * 2 * W + W + i] = DT<T>::from_f(x0[m * W + i]);
  }
}
int concat_rows(cudaStream_t st, int dtype, const float *x, const float *x0, void *out, int M, int W, uint64_t *launches) {
  if (M < 1 || W < 1 || !x || !x0 || !out) return (int)cudaErrorInvalidValue;
  MX_DISPATCH(dtype, (concat_rows_kernel<T><<<M, 256, 0, st>>>(x, x0, reinterpret_cast<T *>(out), W)));
  MX_DONE(1);
}

}  // namespace mx
}  // namespace cake
