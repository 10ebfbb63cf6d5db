// mixers.cu — kernels behind mixers.cuh: latent attention, gated linear recurrences, short convolutions, gated unit norms
// and the routed feed-forward of mixer-list blocks.  sm_100a only.  fp32 everywhere the interface says so; D only where a
// projection, a cache row or a weight is stored.
#include "mixers.cuh"

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <math.h>

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

__device__ __forceinline__ float silu_f(float z) { return z / (1.0f + expf(-z)); }
__device__ __forceinline__ float softplus_f(float z) { return fmaxf(z, 0.f) + log1pf(expf(-fabsf(z))); }

// rotate entry i of a vector whose first `dims` entries are paired (i, i + dims/2); cs / sn: this position's table row
template <typename T>
__device__ __forceinline__ float rotated(const T *v, int i, int dims, const float *cs, const float *sn) {
  const int half = dims >> 1;
  if (i >= dims) return DT<T>::to_f(v[i]);
  if (i < half) return DT<T>::to_f(v[i]) * cs[i] - DT<T>::to_f(v[i + half]) * sn[i];
  return DT<T>::to_f(v[i]) * cs[i - half] + DT<T>::to_f(v[i - half]) * sn[i - half];
}

// ---------------------------------------------------------------------------------------------- latent attention: prep
template <typename T>
__global__ void __launch_bounds__(128) latent_prep_kernel(const LatentPrep p) {
  __shared__ float red[4];
  const int m = blockIdx.x, b = m / p.S, t = m % p.S, pos = p.pos0 + t;
  const T *row = reinterpret_cast<const T *>(p.proj) + (size_t)m * p.ld;
  const T *kv = row + p.kv_col;
  const int Dk = p.rank + p.rot, half = p.rope_dims >> 1;
  const float *cs = p.cos_t + (size_t)pos * half, *sn = p.sin_t + (size_t)pos * half;
  float ss = 0.f;
  for (int i = threadIdx.x; i < p.rank; i += blockDim.x) {
    const float v = DT<T>::to_f(kv[i]);
    ss = fmaf(v, v, ss);
  }
  ss = warp_sum(ss);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
  __syncthreads();
  const float inv = 1.0f / sqrtf((red[0] + red[1] + red[2] + red[3]) / (float)p.rank + p.eps);
  T *crow = reinterpret_cast<T *>(p.cache) + ((size_t)b * p.cap + pos) * Dk;
  const T *w = reinterpret_cast<const T *>(p.norm_w);
  T *ct = p.cache_t ? reinterpret_cast<T *>(p.cache_t) + (size_t)b * p.rank * p.cap_t + pos : nullptr;
  for (int i = threadIdx.x; i < p.rank; i += blockDim.x) {
    const T c = DT<T>::from_f(DT<T>::to_f(kv[i]) * inv * DT<T>::to_f(w[i]));
    crow[i] = c;
    if (ct) ct[(size_t)i * p.cap_t] = c;
  }
  for (int i = threadIdx.x; i < p.rot; i += blockDim.x) crow[p.rank + i] = DT<T>::from_f(rotated<T>(kv + p.rank, i, p.rope_dims, cs, sn));
  T *qa = reinterpret_cast<T *>(p.qa) + (size_t)m * p.heads * Dk;
  for (int i = threadIdx.x; i < p.heads * p.rot; i += blockDim.x) {
    const int h = i / p.rot, r = i % p.rot;
    qa[(size_t)h * Dk + p.rank + r] = DT<T>::from_f(rotated<T>(row + (size_t)h * (p.dim + p.rot) + p.dim, r, p.rope_dims, cs, sn));
  }
}
int latent_prep(cudaStream_t st, int dtype, const LatentPrep &p, uint64_t *launches) {
  MX_DISPATCH(dtype, (latent_prep_kernel<T><<<p.B * p.S, 128, 0, st>>>(p)));
  MX_DONE(1);
}

// ---------------------------------------------------------------------------------------------- latent attention: core
// One warp per (row, head): lanes split the rank + rot columns of a cached row, four keys per round, running softmax.
template <typename T, int NR>
__global__ void __launch_bounds__(128) latent_attn_kernel(const LatentAttn p) {
  const int warp = (int)(((size_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5), lane = threadIdx.x & 31;
  if (warp >= p.B * p.S * p.heads) return;
  const int m = warp / p.heads, h = warp % p.heads, b = m / p.S, t = m % p.S, n_keys = p.pos0 + t + 1;
  const int Dk = p.rank + p.rot;
  const T *q = reinterpret_cast<const T *>(p.qa) + ((size_t)m * p.heads + h) * Dk;
  const T *kc = reinterpret_cast<const T *>(p.cache) + (size_t)b * p.cap * Dk;
  float qv[NR], acc[NR];
#pragma unroll
  for (int i = 0; i < NR; i++) {
    const int c = lane + 32 * i;
    qv[i] = c < Dk ? DT<T>::to_f(q[c]) * p.scale : 0.f;
    acc[i] = 0.f;
  }
  float mx = -INFINITY, l = 0.f;
  for (int j = 0; j < n_keys; j += 4) {
    float kv[4][NR], s[4];
#pragma unroll
    for (int u = 0; u < 4; u++) {
      const bool ok = j + u < n_keys;
      const T *row = kc + (size_t)(ok ? j + u : j) * Dk;
      float part = 0.f;
#pragma unroll
      for (int i = 0; i < NR; i++) {
        const int c = lane + 32 * i;
        kv[u][i] = c < Dk ? DT<T>::to_f(row[c]) : 0.f;
        part = fmaf(qv[i], kv[u][i], part);
      }
      s[u] = part;
    }
#pragma unroll
    for (int u = 0; u < 4; u++) {
      s[u] = warp_sum(s[u]);
      if (j + u >= n_keys) s[u] = -INFINITY;
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
      for (int u = 0; u < 4; u++) a = fmaf(pr[u], kv[u][i], a);
      acc[i] = a;
    }
    mx = mn;
  }
  T *out = reinterpret_cast<T *>(p.lat) + ((size_t)m * p.heads + h) * p.rank;
  const float il = 1.0f / l;
#pragma unroll
  for (int i = 0; i < NR; i++) {
    const int c = lane + 32 * i;
    if (c < p.rank) out[c] = DT<T>::from_f(acc[i] * il);
  }
}
// Steps of a few rows.  CTA (row-head, split): its four warps walk the split's keys four at a time each, their partials are
// merged in shared memory and written as (max, sum, weighted latent); a second kernel merges the splits.
template <typename T, int NR>
__global__ void __launch_bounds__(128) latent_attn_split_kernel(const LatentAttn p) {
  __shared__ float sm_m[4], sm_l[4];
  extern __shared__ float sm_acc[];  // [4][rank]
  const int mh = blockIdx.x, split = blockIdx.y, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m = mh / p.heads, b = m / p.S, t = m % p.S, n_keys = p.pos0 + t + 1, Dk = p.rank + p.rot;
  const int per = ((n_keys + p.nsplit - 1) / p.nsplit + 15) / 16 * 16;
  const int k0 = split * per, k1 = min(n_keys, k0 + per);
  const T *q = reinterpret_cast<const T *>(p.qa) + (size_t)mh * Dk;
  const T *kc = reinterpret_cast<const T *>(p.cache) + (size_t)b * p.cap * Dk;
  float qv[NR], acc[NR];
#pragma unroll
  for (int i = 0; i < NR; i++) {
    const int c = lane + 32 * i;
    qv[i] = c < Dk ? DT<T>::to_f(q[c]) * p.scale : 0.f;
    acc[i] = 0.f;
  }
  float mx = -INFINITY, l = 0.f;
  for (int j = k0 + 4 * warp; j < k1; j += 16) {
    float kv[4][NR], s[4];
#pragma unroll
    for (int u = 0; u < 4; u++) {
      const bool ok = j + u < k1;
      const T *row = kc + (size_t)(ok ? j + u : j) * Dk;
      float part = 0.f;
#pragma unroll
      for (int i = 0; i < NR; i++) {
        const int c = lane + 32 * i;
        kv[u][i] = c < Dk ? DT<T>::to_f(row[c]) : 0.f;
        part = fmaf(qv[i], kv[u][i], part);
      }
      s[u] = part;
    }
#pragma unroll
    for (int u = 0; u < 4; u++) {
      s[u] = warp_sum(s[u]);
      if (j + u >= k1) s[u] = -INFINITY;
    }
    const float mn = fmaxf(fmaxf(mx, fmaxf(s[0], s[1])), fmaxf(s[2], s[3]));
    const float corr = expf(mx - mn);
    float pr[4];
#pragma unroll
    for (int u = 0; u < 4; u++) pr[u] = expf(s[u] - mn);
    l = l * corr + ((pr[0] + pr[1]) + (pr[2] + pr[3]));
#pragma unroll
    for (int i = 0; i < NR; i++) {
      float a = acc[i] * corr;
#pragma unroll
      for (int u = 0; u < 4; u++) a = fmaf(pr[u], kv[u][i], a);
      acc[i] = a;
    }
    mx = mn;
  }
  if (lane == 0) { sm_m[warp] = mx; sm_l[warp] = l; }
#pragma unroll
  for (int i = 0; i < NR; i++) {
    const int c = lane + 32 * i;
    if (c < p.rank) sm_acc[warp * p.rank + c] = acc[i];
  }
  __syncthreads();
  const float M4 = fmaxf(fmaxf(sm_m[0], sm_m[1]), fmaxf(sm_m[2], sm_m[3]));
  float f[4], L = 0.f;
#pragma unroll
  for (int w = 0; w < 4; w++) {
    f[w] = sm_m[w] == -INFINITY ? 0.f : expf(sm_m[w] - M4);
    L = fmaf(sm_l[w], f[w], L);
  }
  float *out = p.part + ((size_t)mh * p.nsplit + split) * (p.rank + 2);
  if (threadIdx.x == 0) { out[0] = M4; out[1] = L; }
  for (int c = threadIdx.x; c < p.rank; c += blockDim.x)
    out[2 + c] = (sm_acc[c] * f[0] + sm_acc[p.rank + c] * f[1]) + (sm_acc[2 * p.rank + c] * f[2] + sm_acc[3 * p.rank + c] * f[3]);
}
template <typename T>
__global__ void __launch_bounds__(128) latent_attn_merge_kernel(const LatentAttn p) {
  const int mh = blockIdx.x;
  const float *part = p.part + (size_t)mh * p.nsplit * (p.rank + 2);
  float M = -INFINITY;
  for (int s = 0; s < p.nsplit; s++) M = fmaxf(M, part[(size_t)s * (p.rank + 2)]);
  float L = 0.f;
  for (int s = 0; s < p.nsplit; s++) {
    const float ms = part[(size_t)s * (p.rank + 2)];
    if (ms != -INFINITY) L = fmaf(part[(size_t)s * (p.rank + 2) + 1], expf(ms - M), L);
  }
  T *out = reinterpret_cast<T *>(p.lat) + (size_t)mh * p.rank;
  for (int c = threadIdx.x; c < p.rank; c += blockDim.x) {
    float a = 0.f;
    for (int s = 0; s < p.nsplit; s++) {
      const float ms = part[(size_t)s * (p.rank + 2)];
      if (ms != -INFINITY) a = fmaf(part[(size_t)s * (p.rank + 2) + 2 + c], expf(ms - M), a);
    }
    out[c] = DT<T>::from_f(a / L);
  }
}

template <typename T> __device__ __forceinline__ void store4(T *d, const float (&v)[4]) {
#pragma unroll
  for (int e = 0; e < 4; e++) d[e] = DT<T>::from_f(v[e]);
}
template <> __device__ __forceinline__ void store4<__nv_bfloat16>(__nv_bfloat16 *d, const float (&v)[4]) {
  *reinterpret_cast<uint2 *>(d) = make_uint2(pack2x<__nv_bfloat16>(v[0], v[1]), pack2x<__nv_bfloat16>(v[2], v[3]));
}
template <> __device__ __forceinline__ void store4<__half>(__half *d, const float (&v)[4]) {
  *reinterpret_cast<uint2 *>(d) = make_uint2(pack2x<__half>(v[0], v[1]), pack2x<__half>(v[2], v[3]));
}
// weights of the matrix-product form: one warp per (token, head) row of the block; kp is a multiple of 128, so a lane
// moves four consecutive scores per load (16 bytes in, 8 + 8 bytes out)
template <typename T>
__global__ void __launch_bounds__(128) latent_softmax_kernel(const LatentSoftmax p) {
  const long row = ((long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (row >= (long)p.n_tok * p.heads) return;
  const int t = (int)(row / p.heads), n_keys = min(p.kp, p.pos_first + t + 1);
  const float4 *s4 = reinterpret_cast<const float4 *>(p.scores + (size_t)row * p.kp);
  T *w = reinterpret_cast<T *>(p.w) + (size_t)row * 2 * p.kp;
  const int n4 = (n_keys + 3) / 4;
  float mxl = -INFINITY, ll = 0.f;  // one read: every lane keeps a running maximum and the sum relative to it
  for (int j4 = lane; j4 < n4; j4 += 32) {
    const float4 v4 = s4[j4];
    const float v[4] = {v4.x * p.scale, v4.y * p.scale, v4.z * p.scale, v4.w * p.scale};
    float m4 = -INFINITY;
#pragma unroll
    for (int e = 0; e < 4; e++)
      if (4 * j4 + e < n_keys) m4 = fmaxf(m4, v[e]);
    if (m4 > mxl) {
      ll *= expf(mxl - m4);
      mxl = m4;
    }
#pragma unroll
    for (int e = 0; e < 4; e++)
      if (4 * j4 + e < n_keys) ll += expf(v[e] - mxl);
  }
  const float mx = warp_max(mxl);
  const float l = warp_sum(mxl == -INFINITY ? 0.f : ll * expf(mxl - mx));
  const float il = 1.0f / l;
  for (int j4 = lane; j4 < p.kp / 4; j4 += 32) {
    float pr[4] = {0.f, 0.f, 0.f, 0.f};
    if (j4 < n4) {
      const float4 v4 = s4[j4];
      const float v[4] = {v4.x, v4.y, v4.z, v4.w};
#pragma unroll
      for (int e = 0; e < 4; e++)
        if (4 * j4 + e < n_keys) pr[e] = expf(fmaf(v[e], p.scale, -mx)) * il;
    }
    float lo[4];
#pragma unroll
    for (int e = 0; e < 4; e++) lo[e] = pr[e] - rnd<T>(pr[e]);
    store4<T>(w + 4 * j4, pr);
    store4<T>(w + p.kp + 4 * j4, lo);
  }
}
int latent_softmax(cudaStream_t st, int dtype, const LatentSoftmax &p, uint64_t *launches) {
  const long warps = (long)p.n_tok * p.heads;
  if (p.kp % 4) return (int)cudaErrorInvalidValue;
  MX_DISPATCH(dtype, (latent_softmax_kernel<T><<<(unsigned)((warps + 3) / 4), 128, 0, st>>>(p)));
  MX_DONE(1);
}

int latent_attention(cudaStream_t st, int dtype, const LatentAttn &p, uint64_t *launches) {
  const int Dk = p.rank + p.rot;
  if (Dk > 32 * 24) return (int)cudaErrorInvalidValue;
  if (p.part && p.nsplit > 1) {
    const dim3 grid((unsigned)(p.B * p.S * p.heads), (unsigned)p.nsplit);
    const size_t smem = (size_t)4 * p.rank * sizeof(float);
    MX_DISPATCH(dtype, {
      if (Dk <= 32 * 6) latent_attn_split_kernel<T, 6><<<grid, 128, smem, st>>>(p);
      else if (Dk <= 32 * 12) latent_attn_split_kernel<T, 12><<<grid, 128, smem, st>>>(p);
      else latent_attn_split_kernel<T, 24><<<grid, 128, smem, st>>>(p);
      latent_attn_merge_kernel<T><<<grid.x, 128, 0, st>>>(p);
    });
    MX_DONE(2);
  }
  const long warps = (long)p.B * p.S * p.heads;
  const unsigned grid = (unsigned)((warps + 3) / 4);
  MX_DISPATCH(dtype, {
    if (Dk <= 32 * 6) latent_attn_kernel<T, 6><<<grid, 128, 0, st>>>(p);
    else if (Dk <= 32 * 12) latent_attn_kernel<T, 12><<<grid, 128, 0, st>>>(p);
    else latent_attn_kernel<T, 24><<<grid, 128, 0, st>>>(p);
  });
  MX_DONE(1);
}

// ---------------------------------------------------------------------------------------------- batched small products
constexpr int HG_BM = 64, HG_BN = 64, HG_BK = 16;
template <typename T>
__global__ void __launch_bounds__(256) head_gemm_kernel(const HeadGemm p) {
  __shared__ float As[HG_BK][HG_BM + 4];
  __shared__ float Ws[HG_BK][HG_BN + 4];
  const int z = blockIdx.z;
  const T *A = reinterpret_cast<const T *>(p.A) + (size_t)z * p.a_zs;
  const T *W = reinterpret_cast<const T *>(p.W) + (size_t)z * p.w_zs;
  T *C = reinterpret_cast<T *>(p.C) + (size_t)z * p.c_zs;
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  const int m0 = blockIdx.y * HG_BM, n0 = blockIdx.x * HG_BN;
  float acc[4][4] = {};
  for (int k0 = 0; k0 < p.K; k0 += HG_BK) {
    for (int i = threadIdx.x; i < HG_BM * HG_BK; i += 256) {
      const int r = i / HG_BK, c = i % HG_BK;
      As[c][r] = (m0 + r < p.M && k0 + c < p.K) ? DT<T>::to_f(A[(size_t)(m0 + r) * p.lda + k0 + c]) : 0.f;
    }
    if (p.w_kn) {
      for (int i = threadIdx.x; i < HG_BN * HG_BK; i += 256) {
        const int c = i / HG_BN, r = i % HG_BN;  // consecutive threads walk n: W[k][n] is contiguous along n
        Ws[c][r] = (n0 + r < p.N && k0 + c < p.K) ? DT<T>::to_f(W[(size_t)(k0 + c) * p.ldw + n0 + r]) : 0.f;
      }
    } else {
      for (int i = threadIdx.x; i < HG_BN * HG_BK; i += 256) {
        const int r = i / HG_BK, c = i % HG_BK;
        Ws[c][r] = (n0 + r < p.N && k0 + c < p.K) ? DT<T>::to_f(W[(size_t)(n0 + r) * p.ldw + k0 + c]) : 0.f;
      }
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < HG_BK; k++) {
      float av[4], wv[4];
#pragma unroll
      for (int i = 0; i < 4; i++) { av[i] = As[k][ty * 4 + i]; wv[i] = Ws[k][tx * 4 + i]; }
#pragma unroll
      for (int i = 0; i < 4; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) acc[i][j] = fmaf(av[i], wv[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; i++) {
    const int m = m0 + ty * 4 + i;
    if (m >= p.M) continue;
#pragma unroll
    for (int j = 0; j < 4; j++) {
      const int n = n0 + tx * 4 + j;
      if (n < p.N) C[(size_t)m * p.ldc + n] = DT<T>::from_f(acc[i][j]);
    }
  }
}
// Steps of a few rows: no tiles.  w_kn (W[z] stored [K, N]): a thread per output column walks k with coalesced loads;
// else (W[z] stored [N, K]): a warp per output column splits k.  The row of A sits in shared memory.
template <typename T>
__global__ void __launch_bounds__(128) head_gemv_kernel(const HeadGemm p) {
  extern __shared__ float arow[];
  const int z = blockIdx.z, m = blockIdx.y;
  const T *A = reinterpret_cast<const T *>(p.A) + (size_t)z * p.a_zs + (size_t)m * p.lda;
  const T *W = reinterpret_cast<const T *>(p.W) + (size_t)z * p.w_zs;
  T *C = reinterpret_cast<T *>(p.C) + (size_t)z * p.c_zs + (size_t)m * p.ldc;
  for (int k = threadIdx.x; k < p.K; k += blockDim.x) arow[k] = DT<T>::to_f(A[k]);
  __syncthreads();
  if (p.w_kn) {
    const int n = blockIdx.x * 128 + threadIdx.x;
    if (n >= p.N) return;
    float a0 = 0.f, a1 = 0.f;
    int k = 0;
    for (; k + 1 < p.K; k += 2) {
      a0 = fmaf(arow[k], DT<T>::to_f(W[(size_t)k * p.ldw + n]), a0);
      a1 = fmaf(arow[k + 1], DT<T>::to_f(W[(size_t)(k + 1) * p.ldw + n]), a1);
    }
    if (k < p.K) a0 = fmaf(arow[k], DT<T>::to_f(W[(size_t)k * p.ldw + n]), a0);
    C[n] = DT<T>::from_f(a0 + a1);
  } else {
    const int n = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (n >= p.N) return;
    const T *w = W + (size_t)n * p.ldw;
    float acc = 0.f;
    for (int k = lane; k < p.K; k += 32) acc = fmaf(arow[k], DT<T>::to_f(w[k]), acc);
    acc = warp_sum(acc);
    if (lane == 0) C[n] = DT<T>::from_f(acc);
  }
}
int head_gemm(cudaStream_t st, int dtype, const HeadGemm &p, uint64_t *launches) {
  if (p.M <= 8 && p.K <= 8192) {
    const dim3 grid(p.w_kn ? (p.N + 127) / 128 : (p.N + 3) / 4, p.M, p.Z);
    MX_DISPATCH(dtype, (head_gemv_kernel<T><<<grid, 128, (size_t)p.K * sizeof(float), st>>>(p)));
    MX_DONE(1);
  }
  dim3 grid((p.N + HG_BN - 1) / HG_BN, (p.M + HG_BM - 1) / HG_BM, p.Z);
  MX_DISPATCH(dtype, (head_gemm_kernel<T><<<grid, 256, 0, st>>>(p)));
  MX_DONE(1);
}

template <typename T>
__global__ void transpose_batched_kernel(const T *__restrict__ in, T *__restrict__ out, int rows, int cols) {
  __shared__ T tile[32][33];
  const size_t z = blockIdx.z;
  const int c0 = blockIdx.x * 32, r0 = blockIdx.y * 32;
  for (int i = threadIdx.y; i < 32; i += blockDim.y)
    if (r0 + i < rows && c0 + (int)threadIdx.x < cols) tile[i][threadIdx.x] = in[(z * rows + r0 + i) * cols + c0 + threadIdx.x];
  __syncthreads();
  for (int i = threadIdx.y; i < 32; i += blockDim.y)
    if (c0 + i < cols && r0 + (int)threadIdx.x < rows) out[(z * cols + c0 + i) * rows + r0 + threadIdx.x] = tile[threadIdx.x][i];
}
int transpose_batched(cudaStream_t st, int dtype, const void *in, void *out, int Z, int rows, int cols, uint64_t *launches) {
  const dim3 grid((cols + 31) / 32, (rows + 31) / 32, Z), block(32, 8);
  MX_DISPATCH(dtype, (transpose_batched_kernel<T><<<grid, block, 0, st>>>(reinterpret_cast<const T *>(in), reinterpret_cast<T *>(out), rows, cols)));
  MX_DONE(1);
}

// ---------------------------------------------------------------------------------------------- gated linear recurrence
// One CTA per (head, batch row) walks the step's tokens in order.  The state sits in shared memory; thread (j, s) owns
// column j of the rows i = s, s + RS, ...: it updates them and adds S[i][j] q[i] to its partial of o[j].
template <typename T>
__global__ void recurrence_kernel(const Recurrence p) {
  extern __shared__ float sm[];
  const int h = blockIdx.x, b = blockIdx.y, dk = p.dk, dv = p.dv;
  const int RS = max(1, (int)blockDim.x / dv);
  float *St = sm, *qs = St + (size_t)dk * dv, *ks = qs + dk, *vs = ks + dk, *part = vs + dv;
  float *gstate = p.state + ((size_t)b * p.heads + h) * dk * dv;
  for (int i = threadIdx.x; i < dk * dv; i += blockDim.x) St[i] = p.pos0 > 0 ? gstate[i] : 0.f;
  const int gcol = (h / p.group_div) * dk, half = p.rope_dims >> 1;
  const T *dtb = reinterpret_cast<const T *>(p.dt_bias), *alog = reinterpret_cast<const T *>(p.a_log), *skp = reinterpret_cast<const T *>(p.skip);
  const float nexpA = p.dt ? -expf(DT<T>::to_f(alog[h])) : 0.f, bias = p.dt ? DT<T>::to_f(dtb[h]) : 0.f;
  const float skip = skp ? DT<T>::to_f(skp[h]) : 0.f;
  const int j = threadIdx.x % dv, s = threadIdx.x / dv;
  const bool owner = s < RS;
  for (int t = 0; t < p.S; t++) {
    const size_t m = (size_t)b * p.S + t;
    const T *qr = reinterpret_cast<const T *>(p.q) + m * p.ldq + gcol;
    const T *kr = reinterpret_cast<const T *>(p.k) + m * p.ldk + gcol;
    const T *vr = reinterpret_cast<const T *>(p.v) + m * p.ldv + (size_t)h * dv;
    float a, bsc;
    if (p.dt) {
      const float d = softplus_f(DT<T>::to_f(reinterpret_cast<const T *>(p.dt)[m * p.lddt + h]) + bias);
      a = expf(nexpA * d);
      bsc = d;
    } else {
      a = p.decay ? p.decay[h] : 1.f;
      bsc = p.kscale;
    }
    if (p.a_tok) {
      a = p.a_tok[m * p.heads + h];
      bsc = p.b_tok[m * p.heads + h];
    }
    const float *cs = p.cos_t ? p.cos_t + (size_t)(p.pos0 + t) * half : nullptr, *sn = p.sin_t ? p.sin_t + (size_t)(p.pos0 + t) * half : nullptr;
    for (int i = threadIdx.x; i < dk; i += blockDim.x) {
      if (cs) {
        qs[i] = rotated<T>(qr, i, p.rope_dims, cs, sn);
        ks[i] = rotated<T>(kr, i, p.rope_dims, cs, sn) * bsc;
      } else {
        qs[i] = DT<T>::to_f(qr[i]);
        ks[i] = DT<T>::to_f(kr[i]) * bsc;
      }
    }
    for (int i = threadIdx.x; i < dv; i += blockDim.x) vs[i] = DT<T>::to_f(vr[i]);
    __syncthreads();
    if (owner) {
      for (int jj = j; jj < dv; jj += blockDim.x) {  // one pass unless dv exceeds the block
        const float v = vs[jj];
        float acc = 0.f;
        for (int i = s; i < dk; i += RS) {
          const float sn_ = fmaf(a, St[(size_t)i * dv + jj], ks[i] * v);
          St[(size_t)i * dv + jj] = sn_;
          acc = fmaf(sn_, qs[i], acc);
        }
        part[(size_t)s * dv + jj] = acc;
      }
    }
    __syncthreads();
    for (int jj = threadIdx.x; jj < dv; jj += blockDim.x) {
      float o = 0.f;
      for (int r = 0; r < RS; r++) o += part[(size_t)r * dv + jj];
      p.o[m * ((size_t)p.heads * dv) + (size_t)h * dv + jj] = fmaf(skip, vs[jj], o);
    }
    __syncthreads();
  }
  for (int i = threadIdx.x; i < dk * dv; i += blockDim.x) gstate[i] = St[i];
}
// The same recurrence for key sizes of 8 R and value sizes that are multiples of 32.  The columns of the state are
// independent, so a CTA owns 32 of them for one (head, batch row): warp s keeps rows s R .. s R + R - 1 of its lanes' columns in
// registers.  Tokens come in chunks of 16: their q, k (rotated, scaled) and v are staged in shared memory once, the 16 updates
// run without a barrier, and the eight warps' partial outputs are added up once per chunk.
constexpr int RC_TT = 16, RC_CB = 32, RC_RS = 8;
template <typename T, int R, bool ROPE>
__global__ void __launch_bounds__(256, R > 16 ? 1 : (ROPE ? 2 : 3)) recurrence_cols_kernel(const Recurrence p) {
  extern __shared__ float sm[];
  constexpr int dk = R * RC_RS;
  float *qs = sm, *ks = qs + RC_TT * dk, *vs = ks + RC_TT * dk, *as = vs + RC_TT * RC_CB, *bs = as + RC_TT, *part = bs + RC_TT;
  const int ncb = p.dv / RC_CB, h = blockIdx.x / ncb, cb = blockIdx.x % ncb, b = blockIdx.y;
  const int lane = threadIdx.x & 31, s = threadIdx.x >> 5;
  float St[R];
  float *gstate = p.state + (((size_t)b * p.heads + h) * dk + (size_t)s * R) * p.dv + cb * RC_CB + lane;
#pragma unroll
  for (int r = 0; r < R; r++) St[r] = p.pos0 > 0 ? gstate[(size_t)r * p.dv] : 0.f;
  const int gcol = (h / p.group_div) * dk, half = p.rope_dims >> 1;
  const T *dtb = reinterpret_cast<const T *>(p.dt_bias), *alog = reinterpret_cast<const T *>(p.a_log), *skp = reinterpret_cast<const T *>(p.skip);
  const float nexpA = p.dt ? -expf(DT<T>::to_f(alog[h])) : 0.f, bias = p.dt ? DT<T>::to_f(dtb[h]) : 0.f;
  const float skip = skp ? DT<T>::to_f(skp[h]) : 0.f;
  // Raw values of the next chunk wait in registers while the current one is computed: (R + 1) / 2 q / k entries (with their
  // rotation partners and table entries), two v entries and one dt per thread.  The loads are straight-line code (indices are
  // clamped, nothing is selected on a loaded value before the chunk is staged), so that they are all in flight at once.
  constexpr int NE = (R + 1) / 2;
  T rq[NE], rqp[NE], rk[NE], rkp[NE], rv[2], rdt = DT<T>::from_f(0.f);
  float rc[NE], rsn[NE];
  const T *dtp = reinterpret_cast<const T *>(p.dt ? p.dt : p.v);  // any valid address when there is no dt
  const int lddt = p.dt ? p.lddt : 0, dth = p.dt ? h : 0;
  auto fetch = [&](int t0) {
    const int nt = min(RC_TT, p.S - t0);
    const size_t m0 = (size_t)b * p.S + t0;
#pragma unroll
    for (int e = 0; e < NE; e++) {
      const int idx = min((int)threadIdx.x + 256 * e, nt * dk - 1), tt = idx / dk, i = idx % dk;
      const T *qr = reinterpret_cast<const T *>(p.q) + (m0 + tt) * p.ldq + gcol;
      const T *kr = reinterpret_cast<const T *>(p.k) + (m0 + tt) * p.ldk + gcol;
      rq[e] = qr[i];
      rk[e] = kr[i];
      if (ROPE) {
        const bool rot = i < p.rope_dims;
        const int ip = rot ? (i < half ? i + half : i - half) : i, it = rot ? (i < half ? i : i - half) : 0;
        rqp[e] = qr[ip];
        rkp[e] = kr[ip];
        rc[e] = p.cos_t[(size_t)(p.pos0 + t0 + tt) * half + it];
        rsn[e] = p.sin_t[(size_t)(p.pos0 + t0 + tt) * half + it];
      }
    }
#pragma unroll
    for (int e = 0; e < 2; e++) {
      const int idx = min((int)threadIdx.x + 256 * e, nt * RC_CB - 1);
      rv[e] = reinterpret_cast<const T *>(p.v)[(m0 + idx / RC_CB) * p.ldv + (size_t)h * p.dv + cb * RC_CB + idx % RC_CB];
    }
    rdt = dtp[(m0 + min((int)threadIdx.x, nt - 1)) * lddt + dth];
  };
  fetch(0);
  for (int t0 = 0; t0 < p.S; t0 += RC_TT) {
    const int nt = min(RC_TT, p.S - t0);
    const size_t m0 = (size_t)b * p.S + t0;
    __syncthreads();  // the previous chunk's outputs have been added up
    if ((int)threadIdx.x < nt) {
      float a = p.decay ? p.decay[h] : 1.f, bsc = p.kscale;
      if (p.dt) {
        const float d = softplus_f(DT<T>::to_f(rdt) + bias);
        a = expf(nexpA * d);
        bsc = d;
      }
      if (p.a_tok) {
        a = p.a_tok[(m0 + threadIdx.x) * p.heads + h];
        bsc = p.b_tok[(m0 + threadIdx.x) * p.heads + h];
      }
      as[threadIdx.x] = a;
      bs[threadIdx.x] = bsc;
    }
#pragma unroll
    for (int e = 0; e < NE; e++) {
      const int idx = threadIdx.x + 256 * e;
      if (idx < nt * dk) {
        float qv = DT<T>::to_f(rq[e]), kv = DT<T>::to_f(rk[e]);
        if (ROPE) {  // entry i of a rotated pair: x_i cos - x_partner sin (first half), x_i cos + x_partner sin (second half)
          const int i = idx % dk;
          if (i < p.rope_dims) {
            const float sn = i < half ? -rsn[e] : rsn[e];
            qv = fmaf(DT<T>::to_f(rqp[e]), sn, qv * rc[e]);
            kv = fmaf(DT<T>::to_f(rkp[e]), sn, kv * rc[e]);
          }
        }
        qs[idx] = qv;
        ks[idx] = kv;
      }
    }
#pragma unroll
    for (int e = 0; e < 2; e++) {
      const int idx = threadIdx.x + 256 * e;
      if (idx < nt * RC_CB) vs[idx] = DT<T>::to_f(rv[e]);
    }
    __syncthreads();
    if (t0 + RC_TT < p.S) fetch(t0 + RC_TT);  // in flight while this chunk is computed
    for (int tt = 0; tt < nt; tt++) {
      const float a = as[tt], v = vs[tt * RC_CB + lane] * bs[tt];
      const float *kq = ks + tt * dk + s * R, *qq = qs + tt * dk + s * R;
      float acc0 = 0.f, acc1 = 0.f;
      if (R % 4 == 0) {
#pragma unroll
        for (int r = 0; r < R; r += 4) {
          const float4 k4 = *reinterpret_cast<const float4 *>(kq + r), q4 = *reinterpret_cast<const float4 *>(qq + r);
          St[r] = fmaf(a, St[r], k4.x * v); acc0 = fmaf(St[r], q4.x, acc0);
          St[r + 1] = fmaf(a, St[r + 1], k4.y * v); acc1 = fmaf(St[r + 1], q4.y, acc1);
          St[r + 2] = fmaf(a, St[r + 2], k4.z * v); acc0 = fmaf(St[r + 2], q4.z, acc0);
          St[r + 3] = fmaf(a, St[r + 3], k4.w * v); acc1 = fmaf(St[r + 3], q4.w, acc1);
        }
      } else {
#pragma unroll
        for (int r = 0; r < R; r += 2) {
          const float2 k2 = *reinterpret_cast<const float2 *>(kq + r), q2 = *reinterpret_cast<const float2 *>(qq + r);
          St[r] = fmaf(a, St[r], k2.x * v); acc0 = fmaf(St[r], q2.x, acc0);
          St[r + 1] = fmaf(a, St[r + 1], k2.y * v); acc1 = fmaf(St[r + 1], q2.y, acc1);
        }
      }
      part[(s * RC_TT + tt) * RC_CB + lane] = acc0 + acc1;
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < nt * RC_CB; idx += 256) {
      const int tt = idx / RC_CB, j = idx % RC_CB;
      float o = 0.f;
#pragma unroll
      for (int w = 0; w < RC_RS; w++) o += part[(w * RC_TT + tt) * RC_CB + j];
      p.o[(m0 + tt) * ((size_t)p.heads * p.dv) + (size_t)h * p.dv + cb * RC_CB + j] = fmaf(skip, vs[idx], o);
    }
  }
#pragma unroll
  for (int r = 0; r < R; r++) gstate[(size_t)r * p.dv] = St[r];
}
template <typename T, int R, bool ROPE> static cudaError_t launch_recurrence_cols2(cudaStream_t st, const Recurrence &p) {
  constexpr int dk = R * RC_RS;
  const size_t smem = (size_t)(2 * RC_TT * dk + RC_TT * RC_CB + 2 * RC_TT + RC_RS * RC_TT * RC_CB) * sizeof(float);
  static int attr_dev = -1;  // per instantiation: the device the attribute was last set on (the value never changes)
  int dev = 0;
  cudaGetDevice(&dev);
  if (smem > 48 * 1024 && attr_dev != dev) {
    cudaError_t e = cudaFuncSetAttribute(recurrence_cols_kernel<T, R, ROPE>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    attr_dev = dev;
  }
  recurrence_cols_kernel<T, R, ROPE><<<dim3(p.heads * (p.dv / RC_CB), p.B), 256, smem, st>>>(p);
  return cudaSuccess;
}
template <typename T, int R> static cudaError_t launch_recurrence_cols(cudaStream_t st, const Recurrence &p) {
  return p.cos_t && p.rope_dims > 0 ? launch_recurrence_cols2<T, R, true>(st, p) : launch_recurrence_cols2<T, R, false>(st, p);
}

int recurrence(cudaStream_t st, int dtype, const Recurrence &p, uint64_t *launches) {
  if (p.dv > 1024 || p.dk < 1) return (int)cudaErrorInvalidValue;
  if (p.dk % RC_RS == 0 && p.dv % RC_CB == 0) {
    cudaError_t e = cudaErrorNotSupported;
    MX_DISPATCH(dtype, {
      switch (p.dk / RC_RS) {
        case 4: e = launch_recurrence_cols<T, 4>(st, p); break;
        case 6: e = launch_recurrence_cols<T, 6>(st, p); break;
        case 8: e = launch_recurrence_cols<T, 8>(st, p); break;
        case 12: e = launch_recurrence_cols<T, 12>(st, p); break;
        case 16: e = launch_recurrence_cols<T, 16>(st, p); break;
        case 24: e = launch_recurrence_cols<T, 24>(st, p); break;
        case 32: e = launch_recurrence_cols<T, 32>(st, p); break;
        default: break;
      }
    });
    if (e == cudaSuccess) MX_DONE(1);
    if (e != cudaErrorNotSupported) return (int)e;
  }
  const int threads = p.dv <= 256 ? 256 : (p.dv + 31) / 32 * 32;
  const int RS = threads / p.dv > 0 ? threads / p.dv : 1;
  const size_t smem = ((size_t)p.dk * p.dv + 2 * p.dk + p.dv + (size_t)RS * p.dv) * sizeof(float);
  if (smem > 227 * 1024) return (int)cudaErrorInvalidValue;
  MX_DISPATCH(dtype, {
    static int attr_dev = -1;
    int dev = 0;
    cudaGetDevice(&dev);
    if (attr_dev != dev) {
      cudaError_t e = cudaFuncSetAttribute(recurrence_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
      if (e != cudaSuccess) return (int)e;
      attr_dev = dev;
    }
    recurrence_kernel<T><<<dim3(p.heads, p.B), threads, smem, st>>>(p);
  });
  MX_DONE(1);
}

// ---------------------------------------------------------------------------------------------- short convolution
template <typename T>
__global__ void __launch_bounds__(256) short_conv_kernel(const ShortConv p) {
  const int m = blockIdx.x, b = m / p.S, t = m % p.S, back = p.taps - 1;
  const T *in = reinterpret_cast<const T *>(p.in);
  const T *w = reinterpret_cast<const T *>(p.w), *bias = reinterpret_cast<const T *>(p.bias);
  const T *hist = reinterpret_cast<const T *>(p.hist) + (size_t)b * back * p.channels;
  T *out = reinterpret_cast<T *>(p.out) + (size_t)m * p.channels;
  for (int ch = blockIdx.y * blockDim.x + threadIdx.x; ch < p.channels; ch += gridDim.y * blockDim.x) {
    float acc = bias ? DT<T>::to_f(bias[ch]) : 0.f;
    for (int jt = 0; jt < p.taps; jt++) {
      const int tt = t - back + jt;
      float x = 0.f;
      if (tt >= 0) x = DT<T>::to_f(in[((size_t)b * p.S + tt) * p.ld + p.col0 + ch]);
      else if (p.pos0 > 0) x = DT<T>::to_f(hist[(size_t)(back + tt) * p.channels + ch]);
      acc = fmaf(DT<T>::to_f(w[(size_t)ch * p.taps + jt]), x, acc);
    }
    out[ch] = DT<T>::from_f(silu_f(acc));
  }
}
// 16-bit D with channel counts, strides and offsets that are multiples of 8: a thread owns eight channels, keeps their
// TAPS x 8 weights and a sliding window of inputs in registers and walks SC_TOK tokens, so that a row is read once
constexpr int SC_TOK = 16;
template <typename T, int TAPS>
__global__ void __launch_bounds__(128) short_conv_vec_kernel(const ShortConv p) {
  const int c8 = blockIdx.y * blockDim.x + threadIdx.x;
  if (c8 >= p.channels / 8) return;
  const int ch = c8 * 8, chunks = (p.S + SC_TOK - 1) / SC_TOK, b = blockIdx.x / chunks, t0 = (blockIdx.x % chunks) * SC_TOK;
  const T *in = reinterpret_cast<const T *>(p.in) + (size_t)b * p.S * p.ld + p.col0 + ch;
  const T *hist = reinterpret_cast<const T *>(p.hist) + (size_t)b * (TAPS - 1) * p.channels + ch;
  T *out = reinterpret_cast<T *>(p.out) + (size_t)b * p.S * p.channels + ch;
  float w[8][TAPS], bias[8], x[TAPS][8];
  {
    const uint4 *w4 = reinterpret_cast<const uint4 *>(reinterpret_cast<const T *>(p.w) + (size_t)ch * TAPS);  // 8 * TAPS contiguous weights
    float tmp[8 * TAPS];
#pragma unroll
    for (int i = 0; i < TAPS; i++) {
      float f[8];
      unpack8<T>(w4[i], f);
#pragma unroll
      for (int e = 0; e < 8; e++) tmp[8 * i + e] = f[e];
    }
#pragma unroll
    for (int e = 0; e < 8; e++)
#pragma unroll
      for (int jt = 0; jt < TAPS; jt++) w[e][jt] = tmp[e * TAPS + jt];
    if (p.bias) unpack8<T>(*reinterpret_cast<const uint4 *>(reinterpret_cast<const T *>(p.bias) + ch), bias);
    else {
#pragma unroll
      for (int e = 0; e < 8; e++) bias[e] = 0.f;
    }
  }
#pragma unroll
  for (int jt = 0; jt < TAPS - 1; jt++) {  // the rows before the chunk: this step's, the history's, or zeros before position 0
    const int tt = t0 - (TAPS - 1) + jt;
    if (tt >= 0) unpack8<T>(*reinterpret_cast<const uint4 *>(in + (size_t)tt * p.ld), x[jt]);
    else if (p.pos0 > 0) unpack8<T>(*reinterpret_cast<const uint4 *>(hist + (size_t)(TAPS - 1 + tt) * p.channels), x[jt]);
    else {
#pragma unroll
      for (int e = 0; e < 8; e++) x[jt][e] = 0.f;
    }
  }
  const int t1 = min(p.S, t0 + SC_TOK);
  for (int t = t0; t < t1; t++) {
    unpack8<T>(*reinterpret_cast<const uint4 *>(in + (size_t)t * p.ld), x[TAPS - 1]);
    float acc[8];
#pragma unroll
    for (int e = 0; e < 8; e++) {
      acc[e] = bias[e];
#pragma unroll
      for (int jt = 0; jt < TAPS; jt++) acc[e] = fmaf(w[e][jt], x[jt][e], acc[e]);
    }
    uint4 o;
    o.x = pack2x<T>(silu_f(acc[0]), silu_f(acc[1])); o.y = pack2x<T>(silu_f(acc[2]), silu_f(acc[3]));
    o.z = pack2x<T>(silu_f(acc[4]), silu_f(acc[5])); o.w = pack2x<T>(silu_f(acc[6]), silu_f(acc[7]));
    *reinterpret_cast<uint4 *>(out + (size_t)t * p.channels) = o;
#pragma unroll
    for (int jt = 0; jt < TAPS - 1; jt++)
#pragma unroll
      for (int e = 0; e < 8; e++) x[jt][e] = x[jt + 1][e];
  }
}
template <typename T> static void launch_short_conv(cudaStream_t st, const ShortConv &p) {
  const bool vec = p.channels % 8 == 0 && p.ld % 8 == 0 && p.col0 % 8 == 0 && p.taps >= 2 && p.taps <= 4 &&
                   (((uintptr_t)p.in | (uintptr_t)p.hist | (uintptr_t)p.out | (uintptr_t)p.bias | (uintptr_t)p.w) & 15) == 0;
  const dim3 gv(p.B * ((p.S + SC_TOK - 1) / SC_TOK), (p.channels / 8 + 127) / 128);
  if (vec && p.taps == 2) short_conv_vec_kernel<T, 2><<<gv, 128, 0, st>>>(p);
  else if (vec && p.taps == 3) short_conv_vec_kernel<T, 3><<<gv, 128, 0, st>>>(p);
  else if (vec && p.taps == 4) short_conv_vec_kernel<T, 4><<<gv, 128, 0, st>>>(p);
  else short_conv_kernel<T><<<dim3(p.B * p.S, (p.channels + 255) / 256), 256, 0, st>>>(p);
}
template <> void launch_short_conv<float>(cudaStream_t st, const ShortConv &p) {
  short_conv_kernel<float><<<dim3(p.B * p.S, (p.channels + 255) / 256), 256, 0, st>>>(p);
}
// after the convolution: the history becomes the last taps - 1 inputs up to the end of this step (zeros before position 0)
template <typename T>
__global__ void short_conv_hist_kernel(const ShortConv p) {
  const int idx = blockIdx.x * blockDim.x + threadIdx.x, back = p.taps - 1;
  if (idx >= p.B * p.channels) return;
  const int b = idx / p.channels, ch = idx % p.channels;
  const T *in = reinterpret_cast<const T *>(p.in);
  T *hist = reinterpret_cast<T *>(p.hist) + (size_t)b * back * p.channels;
  for (int jt = 0; jt < back; jt++) {  // ascending: an entry is read (at jt + S) before it is overwritten
    const int tt = p.S - back + jt;
    T v = DT<T>::from_f(0.f);
    if (tt >= 0) v = in[((size_t)b * p.S + tt) * p.ld + p.col0 + ch];
    else if (p.pos0 > 0) v = hist[(size_t)(jt + p.S) * p.channels + ch];
    hist[(size_t)jt * p.channels + ch] = v;
  }
}
int short_conv(cudaStream_t st, int dtype, const ShortConv &p, uint64_t *launches) {
  MX_DISPATCH(dtype, {
    launch_short_conv<T>(st, p);
    if (p.taps > 1) short_conv_hist_kernel<T><<<(p.B * p.channels + 255) / 256, 256, 0, st>>>(p);
  });
  MX_DONE(p.taps > 1 ? 2 : 1);
}

// ---------------------------------------------------------------------------------------------- gated unit norm
template <typename T> struct Bits16 { typedef T type; };
template <> struct Bits16<float> { typedef __nv_bfloat16 type; };  // never taken for float (sizeof test); keeps the vector path instantiable
template <typename T>
__global__ void __launch_bounds__(128) gate_norm_kernel(const GateNorm p) {
  const long warp = ((long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (warp >= (long)p.M * p.parts) return;
  const int m = (int)(warp / p.parts), g = (int)(warp % p.parts), len = p.n / p.parts, c0 = g * len;
  const float *o = p.o + (size_t)m * p.n + c0;
  const T *gate = reinterpret_cast<const T *>(p.gate) + (size_t)m * p.ldg + c0;
  const T *w = p.w ? reinterpret_cast<const T *>(p.w) + (p.w_period ? 0 : c0) : nullptr;  // w_period == len: every part reads the same gains
  T *out = reinterpret_cast<T *>(p.out) + (size_t)m * p.n + c0;
  const float rdiv = p.row_div ? p.row_div[(size_t)m * p.parts + g] : 1.f;
  const bool sg = p.gate_sigmoid != 0;
  auto gact = [sg](float z) { return sg ? 1.0f / (1.0f + expf(-z)) : silu_f(z); };
  float ss = 0.f;
  // parts whose rows start on 16 bytes: four entries per lane and load
  const bool vec = sizeof(T) == 2 && (len & 3) == 0 && (p.n & 3) == 0 && (p.ldg & 3) == 0 &&
                   (((uintptr_t)p.o | (uintptr_t)p.out) & 15) == 0 && (((uintptr_t)p.gate | (uintptr_t)(p.w ? p.w : p.gate)) & 7) == 0;
  if (vec) {
    const float4 *o4 = reinterpret_cast<const float4 *>(o);
    const uint2 *g2 = reinterpret_cast<const uint2 *>(gate), *w2 = reinterpret_cast<const uint2 *>(w);
    typedef typename Bits16<T>::type B;
    for (int i = lane; i < len / 4; i += 32) {
      const float4 ov = o4[i];
      float v[4] = {ov.x, ov.y, ov.z, ov.w};
      if (p.row_div) { v[0] /= rdiv; v[1] /= rdiv; v[2] /= rdiv; v[3] /= rdiv; }
      if (p.gate_first) {
        const uint2 g = g2[i];
        const float2 ga = DT<B>::unpack2(g.x), gb = DT<B>::unpack2(g.y);
        v[0] *= gact(ga.x); v[1] *= gact(ga.y); v[2] *= gact(gb.x); v[3] *= gact(gb.y);
      }
      ss = fmaf(v[0], v[0], ss); ss = fmaf(v[1], v[1], ss); ss = fmaf(v[2], v[2], ss); ss = fmaf(v[3], v[3], ss);
    }
    ss = warp_sum(ss);
    const float inv = 1.0f / sqrtf(ss / (float)len + p.eps);
    for (int i = lane; i < len / 4; i += 32) {
      const float4 ov = o4[i];
      const uint2 g = g2[i];
      const float2 ga = DT<B>::unpack2(g.x), gb = DT<B>::unpack2(g.y);
      const float gs[4] = {gact(ga.x), gact(ga.y), gact(gb.x), gact(gb.y)};
      float v[4] = {ov.x, ov.y, ov.z, ov.w};
      if (p.row_div) { v[0] /= rdiv; v[1] /= rdiv; v[2] /= rdiv; v[3] /= rdiv; }
      float wv[4] = {1.f, 1.f, 1.f, 1.f};
      if (w) {
        const uint2 ww = w2[i];
        const float2 wa = DT<B>::unpack2(ww.x), wb = DT<B>::unpack2(ww.y);
        wv[0] = wa.x; wv[1] = wa.y; wv[2] = wb.x; wv[3] = wb.y;
      }
#pragma unroll
      for (int e = 0; e < 4; e++) {
        float r = (p.gate_first ? v[e] * gs[e] : v[e]) * inv;
        if (w) r *= wv[e];
        if (!p.gate_first) r *= gs[e];
        v[e] = r;
      }
      *reinterpret_cast<uint2 *>(out + 4 * i) = make_uint2(pack2x<B>(v[0], v[1]), pack2x<B>(v[2], v[3]));
    }
    return;
  }
  for (int i = lane; i < len; i += 32) {
    const float ov = p.row_div ? o[i] / rdiv : o[i];
    const float v = p.gate_first ? ov * gact(DT<T>::to_f(gate[i])) : ov;
    ss = fmaf(v, v, ss);
  }
  ss = warp_sum(ss);
  const float inv = 1.0f / sqrtf(ss / (float)len + p.eps);
  for (int i = lane; i < len; i += 32) {
    const float gs = gact(DT<T>::to_f(gate[i]));
    const float ov = p.row_div ? o[i] / rdiv : o[i];
    float v = (p.gate_first ? ov * gs : ov) * inv;
    if (w) v *= DT<T>::to_f(w[i]);
    if (!p.gate_first) v *= gs;
    out[i] = DT<T>::from_f(v);
  }
}
int gate_norm(cudaStream_t st, int dtype, const GateNorm &p, uint64_t *launches) {
  if (p.parts < 1 || p.n % p.parts || (p.w_period && p.w_period != p.n / p.parts)) return (int)cudaErrorInvalidValue;
  const long warps = (long)p.M * p.parts;
  MX_DISPATCH(dtype, (gate_norm_kernel<T><<<(unsigned)((warps + 3) / 4), 128, 0, st>>>(p)));
  MX_DONE(1);
}

// ---------------------------------------------------------------------------------------------- router
constexpr int MOE_MAX_SLOTS = 8;  // experts + identity <= 256
template <typename T>
__global__ void __launch_bounds__(128) moe_router_kernel(const MoePlan p) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (warp >= p.M) return;
  const int m = warp, E = p.experts + p.identity;
  const float *lg = p.logits + (size_t)m * p.ld;
  const T *corr = reinterpret_cast<const T *>(p.correction);
  float z[MOE_MAX_SLOTS];
#pragma unroll
  for (int sI = 0; sI < MOE_MAX_SLOTS; sI++) {
    z[sI] = lane + 32 * sI < E ? lg[lane + 32 * sI] : -INFINITY;
    if (p.logit_bias && lane + 32 * sI < E) z[sI] += DT<T>::to_f(corr[lane + 32 * sI]);
  }
  float mx = -INFINITY;
#pragma unroll
  for (int sI = 0; sI < MOE_MAX_SLOTS; sI++) mx = fmaxf(mx, z[sI]);
  mx = warp_max(mx);
  float sum = 0.f, sc[MOE_MAX_SLOTS], ch[MOE_MAX_SLOTS];
#pragma unroll
  for (int sI = 0; sI < MOE_MAX_SLOTS; sI++) {
    sc[sI] = lane + 32 * sI < E ? expf(z[sI] - mx) : 0.f;
    sum += sc[sI];
  }
  sum = warp_sum(sum);
#pragma unroll
  for (int sI = 0; sI < MOE_MAX_SLOTS; sI++) {
    const int e = lane + 32 * sI;
    if (p.logit_bias) {  // the choice is by the logits themselves; exp(z - max) / (sum over the chosen) is their softmax
      ch[sI] = z[sI];
      continue;
    }
    sc[sI] = sc[sI] / sum;
    ch[sI] = e < E ? sc[sI] + DT<T>::to_f(corr[e]) : -INFINITY;
  }
  float wsum = 0.f, mine = 0.f;  // lane k keeps the score of the k-th choice
  int mine_id = 0;
  for (int k = 0; k < p.top; k++) {
    float best = -INFINITY, bs = 0.f;
    int bi = 0x7fffffff;
#pragma unroll
    for (int sI = 0; sI < MOE_MAX_SLOTS; sI++)
      if (ch[sI] > best) { best = ch[sI]; bi = lane + 32 * sI; bs = sc[sI]; }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o), os = __shfl_xor_sync(0xffffffffu, bs, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ob > best || (ob == best && oi < bi)) { best = ob; bi = oi; bs = os; }
    }
#pragma unroll
    for (int sI = 0; sI < MOE_MAX_SLOTS; sI++)
      if (bi == lane + 32 * sI) ch[sI] = -INFINITY;
    wsum += bs;
    if (lane == k) { mine = bs; mine_id = bi; }
  }
  if (lane < p.top) {
    p.ids[(size_t)m * p.top + lane] = mine_id;
    p.wts[(size_t)m * p.top + lane] = mine / (wsum + 1e-20f) * p.scale;
  }
  if (p.has_shared_gate && lane == 0) p.sgate[m] = 1.0f / (1.0f + expf(-lg[E]));
}
__global__ void moe_count_kernel(const int *ids, int n, int experts, int *counts) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n && ids[i] < experts) atomicAdd(&counts[ids[i]], 1);
}
// one warp: every expert's pairs start on a multiple of `tile` sorted rows; counts[e] becomes that start (the scatter's cursor)
__global__ void moe_tiles_kernel(const MoePlan p) {
  const int lane = threadIdx.x;
  int done = 0;  // blocks of `tile` rows handed out so far
  for (int base = 0; base < p.experts; base += 32) {
    const int e = base + lane, cnt = e < p.experts ? p.counts[e] : 0, nt = (cnt + p.tile - 1) / p.tile;
    int incl = nt;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int v = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += v;
    }
    const int first = done + incl - nt;
    if (e < p.experts) p.counts[e] = first * p.tile;
    for (int i = 0; i < nt && first + i < p.max_tiles; i++) p.tile_expert[first + i] = e;
    done += __shfl_sync(0xffffffffu, incl, 31);
  }
  for (int i = done + lane; i < p.max_tiles; i += 32) p.tile_expert[i] = -1;
}
__global__ void moe_scatter_kernel(const int *ids, int n, int experts, int *cursor, int *perm, int *pos_of) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n && ids[i] < experts) {
    const int pos = atomicAdd(&cursor[ids[i]], 1);
    perm[pos] = i;
    pos_of[i] = pos;
  }
}
// few (token, slot) pairs (decoding): count, plan and scatter in one CTA with the counters in shared memory
constexpr int MOE_SMALL_PAIRS = 1024;
__global__ void __launch_bounds__(256) moe_plan_small_kernel(const MoePlan p) {
  __shared__ int cnt[32 * MOE_MAX_SLOTS];
  __shared__ int done_s;
  const int ne = p.M * p.top, rows = p.max_tiles * p.tile;
  for (int e = threadIdx.x; e < p.experts; e += blockDim.x) cnt[e] = 0;
  for (int r = threadIdx.x; r < rows; r += blockDim.x) p.perm[r] = -1;
  __syncthreads();
  for (int i = threadIdx.x; i < ne; i += blockDim.x)
    if (p.ids[i] < p.experts) atomicAdd(&cnt[p.ids[i]], 1);
  __syncthreads();
  if (threadIdx.x < 32) {
    const int lane = threadIdx.x;
    int done = 0;
    for (int base = 0; base < p.experts; base += 32) {
      const int e = base + lane, c = e < p.experts ? cnt[e] : 0, nt = (c + p.tile - 1) / p.tile;
      int incl = nt;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int v = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += v;
      }
      const int first = done + incl - nt;
      if (e < p.experts) cnt[e] = first * p.tile;
      for (int i = 0; i < nt && first + i < p.max_tiles; i++) p.tile_expert[first + i] = e;
      done += __shfl_sync(0xffffffffu, incl, 31);
    }
    if (lane == 0) done_s = done;
  }
  __syncthreads();
  for (int i = done_s + threadIdx.x; i < p.max_tiles; i += blockDim.x) p.tile_expert[i] = -1;
  for (int i = threadIdx.x; i < ne; i += blockDim.x)
    if (p.ids[i] < p.experts) {
      const int pos = atomicAdd(&cnt[p.ids[i]], 1);
      p.perm[pos] = i;
      p.pos_of[i] = pos;
    }
}
int moe_route(cudaStream_t st, int dtype, const MoePlan &p, uint64_t *launches) {
  if (p.experts + p.identity > 32 * MOE_MAX_SLOTS || p.top > 32 || p.top < 1 || p.top > p.experts + p.identity) return (int)cudaErrorInvalidValue;
  MX_DISPATCH(dtype, (moe_router_kernel<T><<<(p.M + 3) / 4, 128, 0, st>>>(p)));
  int n = 1;
  if (p.experts > 0 && p.M * p.top <= MOE_SMALL_PAIRS) {
    moe_plan_small_kernel<<<1, 256, 0, st>>>(p);
    n += 1;
  } else if (p.experts > 0) {
    cudaMemsetAsync(p.counts, 0, sizeof(int) * (p.experts + 1), st);
    cudaMemsetAsync(p.perm, 0xff, sizeof(int) * (size_t)p.max_tiles * p.tile, st);
    const int ne = p.M * p.top;
    moe_count_kernel<<<(ne + 255) / 256, 256, 0, st>>>(p.ids, ne, p.experts, p.counts);
    moe_tiles_kernel<<<1, 32, 0, st>>>(p);
    moe_scatter_kernel<<<(ne + 255) / 256, 256, 0, st>>>(p.ids, ne, p.experts, p.counts, p.perm, p.pos_of);
    n += 3;
  }
  MX_DONE(n);
}

template <typename T>
__global__ void __launch_bounds__(128) moe_gather_kernel(const T *__restrict__ h, const int *__restrict__ perm, T *__restrict__ sorted, int W, int top) {
  const size_t r = blockIdx.x;
  const int e = perm[r];
  T *dst = sorted + r * W;
  const T *src = e >= 0 ? h + (size_t)(e / top) * W : nullptr;
  constexpr int VE = 16 / (int)sizeof(T);
  if (W % VE == 0) {
    for (int i = threadIdx.x; i < W / VE; i += blockDim.x)
      reinterpret_cast<uint4 *>(dst)[i] = src ? reinterpret_cast<const uint4 *>(src)[i] : make_uint4(0, 0, 0, 0);
    return;
  }
  for (int i = threadIdx.x; i < W; i += blockDim.x) dst[i] = src ? src[i] : DT<T>::from_f(0.f);
}
int moe_gather(cudaStream_t st, int dtype, const void *h, const int *perm, void *sorted, int rows, int W, int top, uint64_t *launches) {
  MX_DISPATCH(dtype, (moe_gather_kernel<T><<<rows, 128, 0, st>>>(reinterpret_cast<const T *>(h), perm, reinterpret_cast<T *>(sorted), W, top)));
  MX_DONE(1);
}

// ---------------------------------------------------------------------------------------------- experts
// A block of `tile` (= 64) sorted rows shares an expert.  PHASE 0: act = f(Wg h) * (Wu h) into the sorted scratch;
// PHASE 1: y[sorted row] = Wd act.
constexpr int ME_BM = 64, ME_BN = 64, ME_BK = 16;
__device__ __forceinline__ float act_f(float g, int kind) {
  if (kind) return 0.5f * g * (1.0f + tanhf(0.7978845608028654f * g * (1.0f + 0.044715f * g * g)));
  return silu_f(g);
}
template <typename T, int PHASE>
__global__ void __launch_bounds__(256) moe_expert_kernel(const MoeExperts p) {
  const int tl = blockIdx.y, e = p.tile_expert[tl];
  if (e < 0) return;
  __shared__ float As[ME_BK][ME_BM + 4];
  __shared__ float Ws[ME_BK][ME_BN + 4];
  __shared__ float Us[PHASE == 0 ? ME_BK : 1][ME_BN + 4];
  __shared__ int src[ME_BM];
  const int row0 = tl * ME_BM;
  const int K = PHASE == 0 ? p.W : p.ff, N = PHASE == 0 ? p.ff : p.W;
  for (int r = threadIdx.x; r < ME_BM; r += 256) src[r] = p.perm[row0 + r];
  __syncthreads();
  const T *A = PHASE == 0 ? reinterpret_cast<const T *>(p.h) : reinterpret_cast<const T *>(p.act);
  const T *Wa = PHASE == 0 ? reinterpret_cast<const T *>(p.wgu) + (size_t)e * 2 * p.ff * p.W : reinterpret_cast<const T *>(p.wd) + (size_t)e * p.W * p.ff;
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4, n0 = blockIdx.x * ME_BN;
  float acc[4][4] = {}, acu[4][4] = {};
  for (int k0 = 0; k0 < K; k0 += ME_BK) {
    for (int i = threadIdx.x; i < ME_BM * ME_BK; i += 256) {
      const int r = i / ME_BK, c = i % ME_BK;
      float a = 0.f;
      if (src[r] >= 0 && k0 + c < K) {
        const size_t arow = PHASE == 0 ? (size_t)(src[r] / p.top) : (size_t)(row0 + r);
        a = DT<T>::to_f(A[arow * K + k0 + c]);
      }
      As[c][r] = a;
      const bool ok = n0 + r < N && k0 + c < K;
      if (PHASE == 0) {
        Ws[c][r] = ok ? DT<T>::to_f(Wa[(size_t)(2 * (n0 + r)) * K + k0 + c]) : 0.f;
        Us[c][r] = ok ? DT<T>::to_f(Wa[(size_t)(2 * (n0 + r) + 1) * K + k0 + c]) : 0.f;
      } else {
        Ws[c][r] = ok ? DT<T>::to_f(Wa[(size_t)(n0 + r) * K + k0 + c]) : 0.f;
      }
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < ME_BK; k++) {
      float av[4], wv[4], uv[4];
#pragma unroll
      for (int i = 0; i < 4; i++) {
        av[i] = As[k][ty * 4 + i];
        wv[i] = Ws[k][tx * 4 + i];
        uv[i] = PHASE == 0 ? Us[k][tx * 4 + i] : 0.f;
      }
#pragma unroll
      for (int i = 0; i < 4; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) {
          acc[i][j] = fmaf(av[i], wv[j], acc[i][j]);
          if (PHASE == 0) acu[i][j] = fmaf(av[i], uv[j], acu[i][j]);
        }
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; i++) {
    const int r = ty * 4 + i;
    if (src[r] < 0) continue;
#pragma unroll
    for (int j = 0; j < 4; j++) {
      const int n = n0 + tx * 4 + j;
      if (n >= N) continue;
      if (PHASE == 0) {
        if (p.act_kind == 2) {
          reinterpret_cast<T *>(p.act)[(size_t)(row0 + r) * p.ff + n] = DT<T>::from_f(gated_pair<T>(acc[i][j], acu[i][j], 2, p.limit));
          continue;
        }
        const float g = rnd<T>(act_f(rnd<T>(acc[i][j]), p.act_kind));
        reinterpret_cast<T *>(p.act)[(size_t)(row0 + r) * p.ff + n] = DT<T>::from_f(g * rnd<T>(acu[i][j]));
      } else {
        p.y[(size_t)(row0 + r) * p.W + n] = acc[i][j];
      }
    }
  }
}
int moe_experts(cudaStream_t st, int dtype, const MoeExperts &p, uint64_t *launches) {
  if (p.tile != ME_BM) return (int)cudaErrorInvalidValue;
  MX_DISPATCH(dtype, {
    moe_expert_kernel<T, 0><<<dim3((p.ff + ME_BN - 1) / ME_BN, p.max_tiles), 256, 0, st>>>(p);
    moe_expert_kernel<T, 1><<<dim3((p.W + ME_BN - 1) / ME_BN, p.max_tiles), 256, 0, st>>>(p);
  });
  MX_DONE(2);
}

template <typename T>
__global__ void __launch_bounds__(256) moe_combine_kernel(const MoeCombine p) {
  const int m = blockIdx.x;
  const T *h = reinterpret_cast<const T *>(p.h) + (size_t)m * p.W;
  if ((p.W & 3) == 0) {  // 16-byte loads and stores of the fp32 rows
    const float4 *x4 = p.x ? reinterpret_cast<const float4 *>(p.x + (size_t)m * p.W) : nullptr;
    float4 *o4 = reinterpret_cast<float4 *>(p.x_out + (size_t)m * p.W);
    for (int i = blockIdx.y * blockDim.x + threadIdx.x; i < p.W / 4; i += gridDim.y * blockDim.x) {
      float4 s = x4 ? x4[i] : make_float4(0.f, 0.f, 0.f, 0.f);
      for (int k = 0; k < p.top; k++) {
        const size_t pr = (size_t)m * p.top + k;
        const float w = p.wts[pr];
        if (p.ids[pr] < p.experts) {
          const float4 y = reinterpret_cast<const float4 *>(p.y + (size_t)p.pos_of[pr] * p.W)[i];
          s.x = fmaf(w, y.x, s.x); s.y = fmaf(w, y.y, s.y); s.z = fmaf(w, y.z, s.z); s.w = fmaf(w, y.w, s.w);
        } else {
          s.x = fmaf(w, DT<T>::to_f(h[4 * i]), s.x); s.y = fmaf(w, DT<T>::to_f(h[4 * i + 1]), s.y);
          s.z = fmaf(w, DT<T>::to_f(h[4 * i + 2]), s.z); s.w = fmaf(w, DT<T>::to_f(h[4 * i + 3]), s.w);
        }
      }
      o4[i] = s;
    }
    return;
  }
  for (int i = blockIdx.y * blockDim.x + threadIdx.x; i < p.W; i += gridDim.y * blockDim.x) {
    float s = 0.f;
    for (int k = 0; k < p.top; k++) {
      const size_t pr = (size_t)m * p.top + k;
      const int e = p.ids[pr];
      s = fmaf(p.wts[pr], e < p.experts ? p.y[(size_t)p.pos_of[pr] * p.W + i] : DT<T>::to_f(h[i]), s);
    }
    p.x_out[(size_t)m * p.W + i] = (p.x ? p.x[(size_t)m * p.W + i] : 0.f) + s;
  }
}
int moe_combine(cudaStream_t st, int dtype, const MoeCombine &p, uint64_t *launches) {
  MX_DISPATCH(dtype, (moe_combine_kernel<T><<<dim3(p.M, p.M < 64 ? (p.W + 255) / 256 : 1), 256, 0, st>>>(p)));
  MX_DONE(1);
}

// ---------------------------------------------------------------------------------------------- block-wide sums
// sums of up to two values over a CTA of up to 1024 threads; every thread receives the totals
__device__ __forceinline__ void block_sum2(float &a, float &b, float *red /* [64] */) {
  a = warp_sum(a);
  b = warp_sum(b);
  const int w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  __syncthreads();  // red may still be read from a previous use
  if ((threadIdx.x & 31) == 0) { red[w] = a; red[32 + w] = b; }
  __syncthreads();
  float ta = 0.f, tb = 0.f;
  for (int i = 0; i < nw; i++) { ta += red[i]; tb += red[32 + i]; }
  a = ta;
  b = tb;
}

// ---------------------------------------------------------------------------------------------- RMS norm of fp32 rows
template <typename T>
__global__ void __launch_bounds__(256) rms_rows_kernel(const RmsRows p) {
  __shared__ float red[64];
  const int m = blockIdx.x;
  const float *x = p.x + (size_t)m * p.n;
  const T *w = reinterpret_cast<const T *>(p.w);
  float ss = 0.f, z = 0.f;
  for (int i = threadIdx.x; i < p.n; i += blockDim.x) ss = fmaf(x[i], x[i], ss);
  block_sum2(ss, z, red);
  const float inv = 1.0f / sqrtf(ss / (float)p.n + p.eps);
  for (int i = threadIdx.x; i < p.n; i += blockDim.x) {
    const float v = x[i] * inv * (DT<T>::to_f(w[i]) + p.w_add);
    if (p.out32) p.out32[(size_t)m * p.n + i] = v;
    else reinterpret_cast<T *>(p.outD)[(size_t)m * p.n + i] = DT<T>::from_f(v);
  }
}
int rms_rows(cudaStream_t st, int dtype, const RmsRows &p, uint64_t *launches) {
  if (p.M < 1 || p.n < 1 || (!p.out32 && !p.outD)) return (int)cudaErrorInvalidValue;
  MX_DISPATCH(dtype, (rms_rows_kernel<T><<<p.M, 256, 0, st>>>(p)));
  MX_DONE(1);
}

// ---------------------------------------------------------------------------------------------- h + conv(h) over time
template <typename T>
__global__ void __launch_bounds__(256) canon_conv_kernel(const CanonConv p) {
  const int m = blockIdx.x, b = m / p.S, t = m % p.S, back = p.taps - 1;
  const T *w = reinterpret_cast<const T *>(p.w);
  const float *hist = p.hist + (size_t)b * back * p.n;
  for (int ch = blockIdx.y * blockDim.x + threadIdx.x; ch < p.n; ch += gridDim.y * blockDim.x) {
    float acc = p.h[(size_t)m * p.n + ch];
    for (int jt = 0; jt < p.taps; jt++) {
      const int tt = t - back + jt;
      float x = 0.f;
      if (tt >= 0) x = p.h[((size_t)b * p.S + tt) * p.n + ch];
      else if (p.pos0 > 0) x = hist[(size_t)(back + tt) * p.n + ch];
      acc = fmaf(DT<T>::to_f(w[(size_t)ch * p.taps + jt]), x, acc);
    }
    reinterpret_cast<T *>(p.out)[(size_t)m * p.n + ch] = DT<T>::from_f(acc);
  }
}
// widths that are multiples of four with up to eight taps: a thread owns four channels and walks CC_TOK tokens with a sliding
// window of inputs in registers, so that a row of h is read once (16-byte loads) and the output leaves as 8- or 16-byte stores
constexpr int CC_TOK = 16, CC_MAXT = 8;
template <typename T>
__global__ void __launch_bounds__(128) canon_conv_vec_kernel(const CanonConv p) {
  const int c4 = blockIdx.y * blockDim.x + threadIdx.x;
  if (c4 >= p.n / 4) return;
  const int ch = c4 * 4, chunks = (p.S + CC_TOK - 1) / CC_TOK, b = blockIdx.x / chunks, t0 = (blockIdx.x % chunks) * CC_TOK, back = p.taps - 1;
  const T *w = reinterpret_cast<const T *>(p.w);
  const float *h = p.h + (size_t)b * p.S * p.n + ch, *hist = p.hist + (size_t)b * back * p.n + ch;
  float wt[4][CC_MAXT], x[CC_MAXT][4];
#pragma unroll
  for (int e = 0; e < 4; e++)
#pragma unroll
    for (int jt = 0; jt < CC_MAXT; jt++) wt[e][jt] = jt < p.taps ? DT<T>::to_f(w[(size_t)(ch + e) * p.taps + jt]) : 0.f;
  // window slot CC_MAXT - 1 is the current token, slot CC_MAXT - 1 - d the token d back; slots further back than `back` stay zero
#pragma unroll
  for (int d = 1; d < CC_MAXT; d++) {
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (d <= back) {
      const int tt = t0 - d;
      if (tt >= 0) v = *reinterpret_cast<const float4 *>(h + (size_t)tt * p.n);
      else if (p.pos0 > 0) v = *reinterpret_cast<const float4 *>(hist + (size_t)(back + tt) * p.n);
    }
    x[CC_MAXT - 1 - d][0] = v.x; x[CC_MAXT - 1 - d][1] = v.y; x[CC_MAXT - 1 - d][2] = v.z; x[CC_MAXT - 1 - d][3] = v.w;
  }
  const int t1 = min(p.S, t0 + CC_TOK);
  for (int t = t0; t < t1; t++) {
    const float4 v = *reinterpret_cast<const float4 *>(h + (size_t)t * p.n);
    x[CC_MAXT - 1][0] = v.x; x[CC_MAXT - 1][1] = v.y; x[CC_MAXT - 1][2] = v.z; x[CC_MAXT - 1][3] = v.w;
    float acc[4];
#pragma unroll
    for (int e = 0; e < 4; e++) {
      acc[e] = x[CC_MAXT - 1][e];
#pragma unroll
      for (int d = 0; d < CC_MAXT; d++)   // tap index taps - 1 - d multiplies the token d back
        if (d <= back) acc[e] = fmaf(wt[e][back - d], x[CC_MAXT - 1 - d][e], acc[e]);
    }
    store4<T>(reinterpret_cast<T *>(p.out) + ((size_t)b * p.S + t) * p.n + ch, acc);
#pragma unroll
    for (int d = CC_MAXT - 1; d >= 1; d--)
#pragma unroll
      for (int e = 0; e < 4; e++) x[CC_MAXT - 1 - d][e] = x[CC_MAXT - d][e];
  }
}
// afterwards: the history becomes the last taps - 1 inputs up to the end of this step (zeros before position 0)
__global__ void canon_hist_kernel(const CanonConv p) {
  const int idx = blockIdx.x * blockDim.x + threadIdx.x, back = p.taps - 1;
  if (idx >= p.B * p.n) return;
  const int b = idx / p.n, ch = idx % p.n;
  float *hist = p.hist + (size_t)b * back * p.n;
  for (int jt = 0; jt < back; jt++) {  // ascending: an entry is read (at jt + S) before it is overwritten
    const int tt = p.S - back + jt;
    float v = 0.f;
    if (tt >= 0) v = p.h[((size_t)b * p.S + tt) * p.n + ch];
    else if (p.pos0 > 0) v = hist[(size_t)(jt + p.S) * p.n + ch];
    hist[(size_t)jt * p.n + ch] = v;
  }
}
int canon_conv(cudaStream_t st, int dtype, const CanonConv &p, uint64_t *launches) {
  if (p.taps < 1 || p.B < 1 || p.S < 1) return (int)cudaErrorInvalidValue;
  const bool vec = p.n % 4 == 0 && p.taps <= CC_MAXT && (((uintptr_t)p.h | (uintptr_t)p.hist | (uintptr_t)p.out) & 15) == 0;
  MX_DISPATCH(dtype, {
    if (vec) canon_conv_vec_kernel<T><<<dim3(p.B * ((p.S + CC_TOK - 1) / CC_TOK), (p.n / 4 + 127) / 128), 128, 0, st>>>(p);
    else canon_conv_kernel<T><<<dim3(p.B * p.S, (p.n + 255) / 256), 256, 0, st>>>(p);
  });
  if (p.taps > 1) canon_hist_kernel<<<(p.B * p.n + 255) / 256, 256, 0, st>>>(p);
  MX_DONE(p.taps > 1 ? 2 : 1);
}

// ---------------------------------------------------------------------------------------------- sublayer output -> stream
template <typename T>
__global__ void __launch_bounds__(256) branch_merge_kernel(const BranchMerge p) {
  extern __shared__ float ys[];  // [n]
  __shared__ float red[64];
  const int m = blockIdx.x, n = p.n;
  const float *a = p.a + (size_t)m * n, *b = p.b ? p.b + (size_t)m * n : nullptr;
  const T *ba = reinterpret_cast<const T *>(p.a_bias), *bb = reinterpret_cast<const T *>(p.b_bias);
  const T *wa = reinterpret_cast<const T *>(p.wa), *wb = reinterpret_cast<const T *>(p.wb), *post = reinterpret_cast<const T *>(p.post);
  float sa = 0.f, sb = 0.f;
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const float va = a[i] + (ba ? DT<T>::to_f(ba[i]) : 0.f);
    ys[i] = va;
    sa = fmaf(va, va, sa);
    if (b) {
      const float vb = b[i] + (bb ? DT<T>::to_f(bb[i]) : 0.f);
      sb = fmaf(vb, vb, sb);
    }
  }
  float sy = 0.f, z = 0.f;
  if (b) {
    block_sum2(sa, sb, red);
    const float ia = 1.0f / sqrtf(sa / (float)n + p.eps), ib = 1.0f / sqrtf(sb / (float)n + p.eps);
    for (int i = threadIdx.x; i < n; i += blockDim.x) {  // a thread revisits the entries it wrote
      const float vb = b[i] + (bb ? DT<T>::to_f(bb[i]) : 0.f);
      const float y = 0.5f * (ys[i] * ia * DT<T>::to_f(wa[i]) + vb * ib * DT<T>::to_f(wb[i]));
      ys[i] = y;
      sy = fmaf(y, y, sy);
    }
  } else sy = sa;
  float iy = 1.f;
  if (post) {
    block_sum2(sy, z, red);
    iy = 1.0f / sqrtf(sy / (float)n + p.eps);
  }
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const float y = post ? ys[i] * iy * (DT<T>::to_f(post[i]) + p.post_add) : ys[i];
    p.x_out[(size_t)m * n + i] = p.x[(size_t)m * n + i] + y;
  }
}
int branch_merge(cudaStream_t st, int dtype, const BranchMerge &p, uint64_t *launches) {
  if (p.M < 1 || p.n < 1 || !p.a || (p.b && (!p.wa || !p.wb)) || (size_t)p.n * sizeof(float) > 200 * 1024) return (int)cudaErrorInvalidValue;
  const size_t smem = (size_t)p.n * sizeof(float);
  MX_DISPATCH(dtype, {
    if (smem > 48 * 1024) {
      cudaError_t e = cudaFuncSetAttribute(branch_merge_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (e != cudaSuccess) return (int)e;
    }
    branch_merge_kernel<T><<<p.M, 256, smem, st>>>(p);
  });
  MX_DONE(1);
}

// ---------------------------------------------------------------------------------------------- gated delta rule
template <typename T>
__global__ void __launch_bounds__(128) delta_prep_kernel(const DeltaPrep p) {
  const int m = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  const int G = p.kv_heads, dk = p.dk;
  for (int item = warp; item < 2 * G; item += nw) {
    const int which = item / G, hd = item % G;
    const T *src = reinterpret_cast<const T *>(which ? p.k : p.q) + (size_t)m * p.ld + (size_t)hd * dk;
    float *dst = (which ? p.kn : p.qn) + (size_t)m * G * dk + (size_t)hd * dk;
    float ss = 0.f;
    for (int i = lane; i < dk; i += 32) {
      const float v = DT<T>::to_f(src[i]);
      ss = fmaf(v, v, ss);
    }
    ss = warp_sum(ss);
    const float inv = (which ? 1.f : p.qscale) / sqrtf(ss + 1e-6f);
    for (int i = lane; i < dk; i += 32) dst[i] = DT<T>::to_f(src[i]) * inv;
  }
  for (int h = threadIdx.x; h < p.heads; h += blockDim.x) {
    const float br = DT<T>::to_f(reinterpret_cast<const T *>(p.braw)[(size_t)m * p.ldg + h]);
    const float ar = DT<T>::to_f(reinterpret_cast<const T *>(p.araw)[(size_t)m * p.ldg + h]);
    p.beta[(size_t)m * p.heads + h] = 1.0f / (1.0f + expf(-br));
    const float rate = expf(DT<T>::to_f(reinterpret_cast<const T *>(p.a_log)[h]));
    p.g[(size_t)m * p.heads + h] = expf(-rate * softplus_f(ar + DT<T>::to_f(reinterpret_cast<const T *>(p.dt_bias)[h])));
  }
}
int delta_prep(cudaStream_t st, int dtype, const DeltaPrep &p, uint64_t *launches) {
  if (p.M < 1 || p.heads < 1 || p.kv_heads < 1 || p.dk < 1) return (int)cudaErrorInvalidValue;
  MX_DISPATCH(dtype, (delta_prep_kernel<T><<<p.M, 128, 0, st>>>(p)));
  MX_DONE(1);
}

// The columns of the state are independent: u and o of a column need only that column.  Tokens come in chunks of DR_TT whose
// q, k, v, beta and g are staged in shared memory once per CTA (DR_CB columns of one head).
// Register form (dk <= R * RS): RS adjacent lanes share a column, lane s of them keeps rows s R .. s R + R - 1 in registers;
// S^T k and S^T q are R products per lane and log2(RS) shuffles.
constexpr int DR_TT = 16, DR_CB = 32;
template <typename T, int R, int RS>
__global__ void __launch_bounds__(DR_CB * RS) delta_rule_kernel(const DeltaRule p) {
  extern __shared__ float sm[];
  // a lane's slice of a staged q / k row starts R + 4 floats after its neighbour's: the eight 16-byte reads of a quarter-warp
  // then fall into different banks
  constexpr int RP = RS > 1 ? R + 4 : R, ld = RP * RS, NTH = DR_CB * RS;
  float *qs = sm, *ks = qs + DR_TT * ld, *vs = ks + DR_TT * ld, *gs = vs + DR_TT * DR_CB, *bs = gs + DR_TT;
  const int dk = p.dk, dv = p.dv;
  const int ncb = (dv + DR_CB - 1) / DR_CB, h = blockIdx.x / ncb, cb = blockIdx.x % ncb, b = blockIdx.y;
  const int s = threadIdx.x % RS, cl = threadIdx.x / RS, col = cb * DR_CB + cl;
  const bool active = col < dv;
  const int kvh = h / (p.heads / p.kv_heads), qk_ld = p.kv_heads * dk;
  float *gstate = p.state + (((size_t)b * p.heads + h) * dk + (size_t)s * R) * dv + col;
  float St[R];
#pragma unroll
  for (int r = 0; r < R; r++) St[r] = (active && s * R + r < dk && p.pos0 > 0) ? gstate[(size_t)r * dv] : 0.f;
  for (int t0 = 0; t0 < p.S; t0 += DR_TT) {
    const int nt = min(DR_TT, p.S - t0);
    const size_t m0 = (size_t)b * p.S + t0;
    __syncthreads();
    for (int idx = threadIdx.x; idx < nt * R * RS; idx += NTH) {
      const int tt = idx / (R * RS), r = idx % (R * RS), at = tt * ld + (r / R) * RP + r % R;
      qs[at] = r < dk ? p.qn[(m0 + tt) * qk_ld + (size_t)kvh * dk + r] : 0.f;
      ks[at] = r < dk ? p.kn[(m0 + tt) * qk_ld + (size_t)kvh * dk + r] : 0.f;
    }
    for (int idx = threadIdx.x; idx < nt * DR_CB; idx += NTH) {
      const int tt = idx / DR_CB, j = cb * DR_CB + idx % DR_CB;
      vs[idx] = j < dv ? DT<T>::to_f(reinterpret_cast<const T *>(p.v)[(m0 + tt) * p.ldv + (size_t)h * dv + j]) : 0.f;
    }
    if ((int)threadIdx.x < nt) {
      gs[threadIdx.x] = p.g[(m0 + threadIdx.x) * p.heads + h];
      bs[threadIdx.x] = p.beta[(m0 + threadIdx.x) * p.heads + h];
    }
    __syncthreads();
    for (int tt = 0; tt < nt; tt++) {
      const float g = gs[tt];
      const float *kq = ks + tt * ld + s * RP, *qq = qs + tt * ld + s * RP;
      float kr[R];
      float d0 = 0.f, d1 = 0.f;
#pragma unroll
      for (int r = 0; r < R; r += 4) {
        const float4 k4 = *reinterpret_cast<const float4 *>(kq + r);
        kr[r] = k4.x; kr[r + 1] = k4.y; kr[r + 2] = k4.z; kr[r + 3] = k4.w;
        St[r] *= g; d0 = fmaf(St[r], k4.x, d0);
        St[r + 1] *= g; d1 = fmaf(St[r + 1], k4.y, d1);
        St[r + 2] *= g; d0 = fmaf(St[r + 2], k4.z, d0);
        St[r + 3] *= g; d1 = fmaf(St[r + 3], k4.w, d1);
      }
      float d = d0 + d1;
#pragma unroll
      for (int o = RS / 2; o > 0; o >>= 1) d += __shfl_xor_sync(0xffffffffu, d, o);
      const float u = bs[tt] * (vs[tt * DR_CB + cl] - d);
      float o0 = 0.f, o1 = 0.f;
#pragma unroll
      for (int r = 0; r < R; r += 4) {
        const float4 q4 = *reinterpret_cast<const float4 *>(qq + r);
        St[r] = fmaf(kr[r], u, St[r]); o0 = fmaf(St[r], q4.x, o0);
        St[r + 1] = fmaf(kr[r + 1], u, St[r + 1]); o1 = fmaf(St[r + 1], q4.y, o1);
        St[r + 2] = fmaf(kr[r + 2], u, St[r + 2]); o0 = fmaf(St[r + 2], q4.z, o0);
        St[r + 3] = fmaf(kr[r + 3], u, St[r + 3]); o1 = fmaf(St[r + 3], q4.w, o1);
      }
      float o = o0 + o1;
#pragma unroll
      for (int x = RS / 2; x > 0; x >>= 1) o += __shfl_xor_sync(0xffffffffu, o, x);
      if (active && s == 0) p.o[(m0 + tt) * ((size_t)p.heads * dv) + (size_t)h * dv + col] = o;
    }
  }
  if (active) {
#pragma unroll
    for (int r = 0; r < R; r++)
      if (s * R + r < dk) gstate[(size_t)r * dv] = St[r];
  }
}
// Shared-memory form for any dk: a thread owns one column, which sits in shared memory.
template <typename T>
__global__ void __launch_bounds__(DR_CB) delta_rule_smem_kernel(const DeltaRule p) {
  extern __shared__ float sm[];
  const int dk = p.dk, dv = p.dv, ld = (dk + 3) / 4 * 4;
  float *qs = sm, *ks = qs + DR_TT * ld, *vs = ks + DR_TT * ld, *gs = vs + DR_TT * DR_CB, *bs = gs + DR_TT, *Ss = bs + DR_TT;
  const int ncb = (dv + DR_CB - 1) / DR_CB, h = blockIdx.x / ncb, cb = blockIdx.x % ncb, b = blockIdx.y;
  const int col = cb * DR_CB + threadIdx.x;
  const bool active = col < dv;
  const int kvh = h / (p.heads / p.kv_heads), qk_ld = p.kv_heads * dk;
  float *gstate = p.state + ((size_t)b * p.heads + h) * dk * dv + col;
  for (int r = 0; r < dk; r++) Ss[r * DR_CB + threadIdx.x] = (active && p.pos0 > 0) ? gstate[(size_t)r * dv] : 0.f;
  for (int t0 = 0; t0 < p.S; t0 += DR_TT) {
    const int nt = min(DR_TT, p.S - t0);
    const size_t m0 = (size_t)b * p.S + t0;
    __syncthreads();
    for (int idx = threadIdx.x; idx < nt * ld; idx += DR_CB) {
      const int tt = idx / ld, r = idx % ld;
      qs[idx] = r < dk ? p.qn[(m0 + tt) * qk_ld + (size_t)kvh * dk + r] : 0.f;
      ks[idx] = r < dk ? p.kn[(m0 + tt) * qk_ld + (size_t)kvh * dk + r] : 0.f;
    }
    for (int idx = threadIdx.x; idx < nt * DR_CB; idx += DR_CB) {
      const int tt = idx / DR_CB, j = cb * DR_CB + idx % DR_CB;
      vs[idx] = j < dv ? DT<T>::to_f(reinterpret_cast<const T *>(p.v)[(m0 + tt) * p.ldv + (size_t)h * dv + j]) : 0.f;
    }
    if ((int)threadIdx.x < nt) {
      gs[threadIdx.x] = p.g[(m0 + threadIdx.x) * p.heads + h];
      bs[threadIdx.x] = p.beta[(m0 + threadIdx.x) * p.heads + h];
    }
    __syncthreads();
    for (int tt = 0; tt < nt; tt++) {
      const float g = gs[tt];
      const float *kq = ks + tt * ld, *qq = qs + tt * ld;
      float d = 0.f;
      for (int r = 0; r < dk; r++) {
        const float sv = Ss[r * DR_CB + threadIdx.x] * g;
        Ss[r * DR_CB + threadIdx.x] = sv;
        d = fmaf(sv, kq[r], d);
      }
      const float u = bs[tt] * (vs[tt * DR_CB + threadIdx.x] - d);
      float o = 0.f;
      for (int r = 0; r < dk; r++) {
        const float sv = fmaf(kq[r], u, Ss[r * DR_CB + threadIdx.x]);
        Ss[r * DR_CB + threadIdx.x] = sv;
        o = fmaf(sv, qq[r], o);
      }
      if (active) p.o[(m0 + tt) * ((size_t)p.heads * dv) + (size_t)h * dv + col] = o;
    }
  }
  if (active)
    for (int r = 0; r < dk; r++) gstate[(size_t)r * dv] = Ss[r * DR_CB + threadIdx.x];
}
template <typename T, int R, int RS> static cudaError_t launch_delta_rule(cudaStream_t st, const DeltaRule &p) {
  const size_t smem = ((size_t)2 * DR_TT * (RS > 1 ? R + 4 : R) * RS + (size_t)DR_TT * DR_CB + 2 * DR_TT) * sizeof(float);
  delta_rule_kernel<T, R, RS><<<dim3(p.heads * ((p.dv + DR_CB - 1) / DR_CB), p.B), DR_CB * RS, smem, st>>>(p);
  return cudaSuccess;
}
template <typename T> static cudaError_t launch_delta_rule_smem(cudaStream_t st, const DeltaRule &p) {
  const int ld = (p.dk + 3) / 4 * 4;
  const size_t smem = ((size_t)2 * DR_TT * ld + (size_t)DR_TT * DR_CB + 2 * DR_TT + (size_t)p.dk * DR_CB) * sizeof(float);
  if (smem > 200 * 1024) return cudaErrorInvalidValue;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(delta_rule_smem_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
  }
  delta_rule_smem_kernel<T><<<dim3(p.heads * ((p.dv + DR_CB - 1) / DR_CB), p.B), DR_CB, smem, st>>>(p);
  return cudaSuccess;
}
int delta_rule(cudaStream_t st, int dtype, const DeltaRule &p, uint64_t *launches) {
  if (p.B < 1 || p.S < 1 || p.heads < 1 || p.kv_heads < 1 || p.heads % p.kv_heads || p.dk < 1 || p.dv < 1) return (int)cudaErrorInvalidValue;
  cudaError_t e = cudaSuccess;
  MX_DISPATCH(dtype, {
    if (p.dk <= 16) e = launch_delta_rule<T, 16, 1>(st, p);
    else if (p.dk <= 32) e = launch_delta_rule<T, 16, 2>(st, p);
    else if (p.dk <= 64) e = launch_delta_rule<T, 16, 4>(st, p);
    else if (p.dk <= 128) e = launch_delta_rule<T, 16, 8>(st, p);
    else if (p.dk <= 256) e = launch_delta_rule<T, 32, 8>(st, p);
    else e = launch_delta_rule_smem<T>(st, p);
  });
  if (e != cudaSuccess) return (int)e;
  MX_DONE(1);
}

// ---------------------------------------------------------------------------------------------- exponential gates
// One CTA of four warps per (head, batch row) walks the tokens in chunks of 32.  All threads stage the chunk's q and k; warp 0
// computes the chunk's log gates (a lane per token), then the running maximum as a prefix scan: m' = max(f + m, i) composes as
// (f1, i1) then (f2, i2) = (f1 + f2, max(f2 + i1, i2)); then it walks the tokens: lane l owns the entries l, l + 32, ... of n.
constexpr int GP_TT = 32, GP_THREADS = 128, GP_NE = 8;
template <typename T>
__global__ void __launch_bounds__(GP_THREADS) gate_prep_kernel(const GatePrep p) {
  extern __shared__ float sm[];
  const int h = blockIdx.x, b = blockIdx.y, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, dk = p.dk;
  float *ns = sm, *ks = ns + dk, *qs = ks + GP_TT * dk, *as = qs + GP_TT * dk, *bs = as + GP_TT, *es = bs + GP_TT, *dots = es + GP_TT;
  float *aux = p.aux + ((size_t)b * p.heads + h) * (dk + 1);
  if (warp == 0)
    for (int r = lane; r < dk; r += 32) ns[r] = p.pos0 > 0 ? aux[r] : 0.f;
  float mx = p.pos0 > 0 ? aux[dk] : 0.f;   // warp 0 carries it
  const float ib = DT<T>::to_f(reinterpret_cast<const T *>(p.i_b)[h]), fb = DT<T>::to_f(reinterpret_cast<const T *>(p.f_b)[h]);
  const bool vec = sizeof(T) == 2 && (dk & 7) == 0 && (p.ld & 7) == 0 && (((uintptr_t)p.q | (uintptr_t)p.k) & 15) == 0;
  for (int t0 = 0; t0 < p.S; t0 += GP_TT) {
    const int nt = min(GP_TT, p.S - t0);
    const size_t m0 = (size_t)b * p.S + t0;
    __syncthreads();   // the previous chunk has been consumed
    if (vec) {
      typedef typename Bits16<T>::type B;
      const int c8 = dk / 8;
      for (int base = threadIdx.x; base < nt * c8; base += 4 * GP_THREADS) {  // eight 16-byte loads in flight per thread
        uint4 rk[4], rq[4];
#pragma unroll
        for (int u = 0; u < 4; u++) {
          const int idx = min(base + u * GP_THREADS, nt * c8 - 1), tt = idx / c8, r = (idx % c8) * 8;
          rk[u] = *reinterpret_cast<const uint4 *>(reinterpret_cast<const T *>(p.k) + (m0 + tt) * p.ld + (size_t)h * dk + r);
          rq[u] = *reinterpret_cast<const uint4 *>(reinterpret_cast<const T *>(p.q) + (m0 + tt) * p.ld + (size_t)h * dk + r);
        }
#pragma unroll
        for (int u = 0; u < 4; u++) {
          const int idx = base + u * GP_THREADS;
          if (idx < nt * c8) {
            const int tt = idx / c8, r = (idx % c8) * 8;
            float f[8];
            unpack8<B>(rk[u], f);
#pragma unroll
            for (int e = 0; e < 8; e++) ks[tt * dk + r + e] = f[e];
            unpack8<B>(rq[u], f);
#pragma unroll
            for (int e = 0; e < 8; e++) qs[tt * dk + r + e] = f[e];
          }
        }
      }
    } else {
      for (int idx = threadIdx.x; idx < nt * dk; idx += GP_THREADS) {
        const int tt = idx / dk, r = idx % dk;
        ks[idx] = DT<T>::to_f(reinterpret_cast<const T *>(p.k)[(m0 + tt) * p.ld + (size_t)h * dk + r]);
        qs[idx] = DT<T>::to_f(reinterpret_cast<const T *>(p.q)[(m0 + tt) * p.ld + (size_t)h * dk + r]);
      }
    }
    if (warp == 0) {
      float li = -INFINITY, lf = 0.f;   // tokens past the chunk's end: the identity of the composition
      if (lane < nt) {
        const float ir = DT<T>::to_f(reinterpret_cast<const T *>(p.iraw)[(m0 + lane) * p.ldg + h]) + ib;
        const float fr = DT<T>::to_f(reinterpret_cast<const T *>(p.fraw)[(m0 + lane) * p.ldg + h]) + fb;
        li = p.cap * tanhf(ir / p.cap);
        const float z = p.cap * tanhf(fr / p.cap);
        lf = fminf(z, 0.f) - log1pf(expf(-fabsf(z)));  // log sigmoid(z)
      }
      float F = lf, I = li;   // inclusive scan of (F, I) over the lanes
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const float Fp = __shfl_up_sync(0xffffffffu, F, o), Ip = __shfl_up_sync(0xffffffffu, I, o);
        if (lane >= o) {
          I = fmaxf(F + Ip, I);
          F = Fp + F;
        }
      }
      const float mt = fmaxf(F + mx, I);
      float mp = __shfl_up_sync(0xffffffffu, mt, 1);
      if (lane == 0) mp = mx;
      if (lane < nt) {
        as[lane] = expf(lf + mp - mt);
        bs[lane] = expf(li - mt);
        es[lane] = expf(-mt);
      }
      mx = __shfl_sync(0xffffffffu, mt, nt - 1);
    }
    __syncthreads();
    if (warp == 0) {
      const bool in_regs = dk <= 32 * GP_NE;   // the lane's entries of n stay in registers over the chunk
      float nr[GP_NE];
#pragma unroll
      for (int e = 0; e < GP_NE; e++) nr[e] = (in_regs && lane + 32 * e < dk) ? ns[lane + 32 * e] : 0.f;
      for (int tt = 0; tt < nt; tt++) {
        const float a = as[tt], bb = bs[tt];
        float dot = 0.f;
        if (in_regs) {
#pragma unroll
          for (int e = 0; e < GP_NE; e++) {
            const int r = min(lane + 32 * e, dk - 1);
            nr[e] = fmaf(a, nr[e], bb * ks[tt * dk + r]);
            dot = fmaf(lane + 32 * e < dk ? nr[e] : 0.f, qs[tt * dk + r], dot);
          }
        } else {
          for (int r = lane; r < dk; r += 32) {
            const float nv = fmaf(a, ns[r], bb * ks[tt * dk + r]);
            ns[r] = nv;
            dot = fmaf(nv, qs[tt * dk + r], dot);
          }
        }
        dots[tt * 32 + lane] = dot;   // the lanes' parts of n . q: added up after the walk, off its critical path
      }
      if (in_regs) {
#pragma unroll
        for (int e = 0; e < GP_NE; e++)
          if (lane + 32 * e < dk) ns[lane + 32 * e] = nr[e];
      }
    }
    __syncthreads();
    for (int tt = warp; tt < nt; tt += GP_THREADS / 32) {
      const float dot = warp_sum(dots[tt * 32 + lane]) * p.qscale;
      if (lane == 0) {
        const size_t o = (m0 + tt) * p.heads + h;
        p.a[o] = as[tt];
        p.b[o] = bs[tt];
        p.div[o] = (fmaxf(fabsf(dot), es[tt]) + 1e-6f) / p.qscale;
      }
    }
  }
  if (warp == 0) {
    __syncwarp();
    for (int r = lane; r < dk; r += 32) aux[r] = ns[r];
    if (lane == 0) aux[dk] = mx;
  }
}
int gate_prep(cudaStream_t st, int dtype, const GatePrep &p, uint64_t *launches) {
  if (p.B < 1 || p.S < 1 || p.heads < 1 || p.dk < 1 || !(p.cap > 0.f) || !(p.qscale > 0.f)) return (int)cudaErrorInvalidValue;
  const size_t smem = ((size_t)p.dk * (1 + 2 * GP_TT) + 3 * GP_TT + 32 * GP_TT) * sizeof(float);
  if (smem > 200 * 1024) return (int)cudaErrorInvalidValue;
  MX_DISPATCH(dtype, {
    if (smem > 48 * 1024) {
      cudaError_t e = cudaFuncSetAttribute(gate_prep_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (e != cudaSuccess) return (int)e;
    }
    gate_prep_kernel<T><<<dim3(p.heads, p.B), GP_THREADS, smem, st>>>(p);
  });
  MX_DONE(1);
}

// ---------------------------------------------------------------------------------------------- attention with mixed heads
// Scores of one key against up to eight query heads of its kv head: acc[i] = q_i . k
template <typename T>
__device__ __forceinline__ void key_scores8(const T *__restrict__ krow, const float *__restrict__ q, int ng, int dim, float (&acc)[8]) {
#pragma unroll
  for (int i = 0; i < 8; i++) acc[i] = 0.f;
  if (sizeof(T) == 2 && (dim & 7) == 0 && ((uintptr_t)krow & 15) == 0) {
    typedef typename Bits16<T>::type B;
    for (int d0 = 0; d0 < dim; d0 += 32) {   // four 16-byte loads of the key row in flight
      uint4 kr[4];
#pragma unroll
      for (int u = 0; u < 4; u++) kr[u] = *reinterpret_cast<const uint4 *>(krow + min(d0 + 8 * u, dim - 8));
#pragma unroll
      for (int u = 0; u < 4; u++) {
        const int d = d0 + 8 * u;
        if (d < dim) {
          float kf[8];
          unpack8<B>(kr[u], kf);
#pragma unroll
          for (int i = 0; i < 8; i++)
            if (i < ng) {
              const float4 qa = *reinterpret_cast<const float4 *>(q + i * dim + d), qb = *reinterpret_cast<const float4 *>(q + i * dim + d + 4);
              float s = acc[i];
              s = fmaf(kf[0], qa.x, s); s = fmaf(kf[1], qa.y, s); s = fmaf(kf[2], qa.z, s); s = fmaf(kf[3], qa.w, s);
              s = fmaf(kf[4], qb.x, s); s = fmaf(kf[5], qb.y, s); s = fmaf(kf[6], qb.z, s); s = fmaf(kf[7], qb.w, s);
              acc[i] = s;
            }
        }
      }
    }
    return;
  }
  for (int d = 0; d < dim; d++) {
    const float kv = DT<T>::to_f(krow[d]);
#pragma unroll
    for (int i = 0; i < 8; i++)
      if (i < ng) acc[i] = fmaf(kv, q[i * dim + d], acc[i]);
  }
}

// One CTA per query row (and per key range when the keys are split), all heads.  A thread works on one (key, key head) pair of a
// tile of KT = blockDim / kv_heads keys: it computes the scores of that key head's query heads.  Pass 1: every thread keeps a
// running (max, sum) per head over its keys, merged per head at the end.  Pass 2: the scores are computed again and normalised;
// after a barrier the thread mixes the weights of its key for its key head's heads across all heads, and after another the tile
// of mixed weights in shared memory is applied to the values by threads that own output entries (eight adjacent ones and
// 16-byte value loads where the sizes allow).
// PHASE 0: both passes in one kernel.  PHASE 1 / 2: the passes of the split form (stats of a key range -> part; the second
// pass merges the ranges' stats itself and leaves partial outputs in part).
constexpr int TA_MAXO = 16;
template <typename T, int PHASE>
__global__ void __launch_bounds__(256) talk_attn_kernel(const TalkAttn p) {
  extern __shared__ float sm[];
  const int NT = blockDim.x, H = p.heads, G = p.kv_heads, dim = p.dim, vdim = p.vdim, grp = H / G;
  float *qs = sm, *M_ = qs + (size_t)H * dim, *L_ = M_ + H, *tk = L_ + H, *ta = tk + H * H, *tb = ta + (size_t)H * NT;
  const int m = blockIdx.x, b = m / p.S, t = m % p.S, pos = p.pos0 + t, nk_all = pos + 1;
  const int ns = PHASE == 0 ? 1 : p.nsplit, sp = PHASE == 0 ? 0 : blockIdx.y;
  const int per = (nk_all + ns - 1) / ns, k_lo = sp * per, k_hi = min(nk_all, k_lo + per);
  const T *kc = reinterpret_cast<const T *>(p.kc) + (size_t)b * G * p.cap * dim;
  const T *vc = reinterpret_cast<const T *>(p.vc) + (size_t)b * G * p.cap * vdim;
  for (int i = threadIdx.x; i < H * dim; i += NT) qs[i] = DT<T>::to_f(reinterpret_cast<const T *>(p.q)[(size_t)m * p.ldq + i]);
  if (p.talk)
    for (int i = threadIdx.x; i < H * H; i += NT) tk[i] = DT<T>::to_f(reinterpret_cast<const T *>(p.talk)[i]);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = NT >> 5;
  const int KT = NT / G, kl = threadIdx.x % KT, c = threadIdx.x / KT;   // this thread's key slot and key head (c >= G: idle)
  if (PHASE != 2) {
    for (int g = 0; g < H; g++) { ta[(size_t)g * NT + threadIdx.x] = -INFINITY; tb[(size_t)g * NT + threadIdx.x] = 0.f; }
    __syncthreads();  // qs, and the initial stats
    if (c < G)
      for (int j = k_lo + kl; j < k_hi; j += KT) {
        const int dist = min(pos - j, p.bias_len - 1);
        const T *krow = kc + ((size_t)c * p.cap + j) * dim;
        for (int g0 = 0; g0 < grp; g0 += 8) {
          const int ng = min(8, grp - g0), gb = c * grp + g0;
          float acc[8];
          key_scores8<T>(krow, qs + (size_t)gb * dim, ng, dim, acc);
#pragma unroll
          for (int i = 0; i < 8; i++)
            if (i < ng) {
              const float s = fmaf(acc[i], p.scale, p.bias ? p.bias[(size_t)dist * H + gb + i] : 0.f);
              const size_t o = (size_t)(gb + i) * NT + kl;   // slot kl of head gb + i: only this thread touches it
              const float mo = ta[o], mn = fmaxf(mo, s);
              tb[o] = tb[o] * expf(mo - mn) + expf(s - mn);  // exp(-inf) = 0 on the first key
              ta[o] = mn;
            }
        }
      }
    __syncthreads();
    for (int g = warp; g < H; g += nw) {  // merge the slots of head g
      float mx = -INFINITY;
      for (int i = lane; i < KT; i += 32) mx = fmaxf(mx, ta[(size_t)g * NT + i]);
      mx = warp_max(mx);
      float l = 0.f;
      for (int i = lane; i < KT; i += 32) {
        const float mi = ta[(size_t)g * NT + i];
        if (mi > -INFINITY) l += tb[(size_t)g * NT + i] * expf(mi - mx);
      }
      l = warp_sum(l);
      if (lane == 0) {
        if (PHASE == 1) {
          float *st = p.part + (((size_t)m * ns + sp) * H + g) * 2;
          st[0] = mx;
          st[1] = l;
        } else { M_[g] = mx; L_[g] = l; }
      }
    }
    if (PHASE == 1) return;
    __syncthreads();
  } else {
    for (int g = threadIdx.x; g < H; g += NT) {  // merge the key ranges' stats
      float mx = -INFINITY;
      for (int s2 = 0; s2 < ns; s2++) mx = fmaxf(mx, p.part[(((size_t)m * ns + s2) * H + g) * 2]);
      float l = 0.f;
      for (int s2 = 0; s2 < ns; s2++) {
        const float *st = p.part + (((size_t)m * ns + s2) * H + g) * 2;
        if (st[0] > -INFINITY) l += st[1] * expf(st[0] - mx);
      }
      M_[g] = mx;
      L_[g] = l;
    }
    __syncthreads();
  }
  // pass 2, once per TA_MAXO * NT output entries (one round unless heads * vdim exceeds that)
  const int n_out = H * vdim;
  const bool vec = sizeof(T) == 2 && (vdim & 7) == 0 && (((uintptr_t)p.vc) & 15) == 0;   // eight adjacent entries per work item
  const int n_items = vec ? n_out / 8 : n_out, per_round = vec ? (TA_MAXO / 8) * NT : TA_MAXO * NT;
  for (int o0 = 0; o0 < n_items; o0 += per_round) {
    float acc[TA_MAXO];
#pragma unroll
    for (int k = 0; k < TA_MAXO; k++) acc[k] = 0.f;
    for (int j0 = k_lo; j0 < k_hi; j0 += KT) {
      const int j = j0 + kl, nj = min(KT, k_hi - j0);
      const bool mine = c < G && j < k_hi;
      if (mine) {
        const int dist = min(pos - j, p.bias_len - 1);
        const T *krow = kc + ((size_t)c * p.cap + j) * dim;
        for (int g0 = 0; g0 < grp; g0 += 8) {
          const int ng = min(8, grp - g0), gb = c * grp + g0;
          float sc[8];
          key_scores8<T>(krow, qs + (size_t)gb * dim, ng, dim, sc);
#pragma unroll
          for (int i = 0; i < 8; i++)
            if (i < ng) {
              const float s = fmaf(sc[i], p.scale, p.bias ? p.bias[(size_t)dist * H + gb + i] : 0.f);
              ta[(size_t)(gb + i) * NT + kl] = expf(s - M_[gb + i]) / L_[gb + i];
            }
        }
      }
      if (p.talk) {
        __syncthreads();   // the weights of every head for this tile's keys
        if (mine)
          for (int hh = c * grp; hh < (c + 1) * grp; hh++) {
            float wv = 0.f;
            for (int g = 0; g < H; g++) wv = fmaf(tk[hh * H + g], ta[(size_t)g * NT + kl], wv);
            tb[(size_t)hh * NT + kl] = wv;
          }
      }
      __syncthreads();
      const float *wt = p.talk ? tb : ta;
      if (vec) {
        typedef typename Bits16<T>::type B;
#pragma unroll
        for (int k = 0; k < TA_MAXO / 8; k++) {
          const int it = o0 + threadIdx.x + k * NT;
          if (it < n_items) {
            const int hh = (it * 8) / vdim, e = (it * 8) % vdim;
            const T *vcol = vc + ((size_t)(hh / grp) * p.cap + j0) * vdim + e;
            const float *wrow = wt + (size_t)hh * NT;
            for (int jj = 0; jj < nj; jj++) {
              float vf[8];
              unpack8<B>(*reinterpret_cast<const uint4 *>(vcol + (size_t)jj * vdim), vf);
              const float wj = wrow[jj];
#pragma unroll
              for (int x = 0; x < 8; x++) acc[8 * k + x] = fmaf(wj, vf[x], acc[8 * k + x]);
            }
          }
        }
      } else {
#pragma unroll
        for (int k = 0; k < TA_MAXO; k++) {
          const int idx = o0 + threadIdx.x + k * NT;
          if (idx < n_out) {
            const int hh = idx / vdim, e = idx % vdim;
            const T *vcol = vc + ((size_t)(hh / grp) * p.cap + j0) * vdim + e;
            const float *wrow = wt + (size_t)hh * NT;
            float a = acc[k];
            for (int jj = 0; jj < nj; jj++) a = fmaf(wrow[jj], DT<T>::to_f(vcol[(size_t)jj * vdim]), a);
            acc[k] = a;
          }
        }
      }
      __syncthreads();
    }
#pragma unroll
    for (int k = 0; k < TA_MAXO; k++) {
      // the output entry of accumulator k: eight adjacent ones per work item in the vector form
      const int idx = vec ? (o0 + threadIdx.x + (k / 8) * NT) * 8 + k % 8 : o0 + threadIdx.x + k * NT;
      const bool live = vec ? (o0 + threadIdx.x + (k / 8) * NT) < n_items : idx < n_out;
      if (live) {
        if (PHASE == 2) {
          p.part[(size_t)p.B * p.S * ns * H * 2 + ((size_t)m * ns + sp) * n_out + idx] = acc[k];
        } else {
          float o = acc[k];
          if (p.gate) o *= 1.0f / (1.0f + expf(-DT<T>::to_f(reinterpret_cast<const T *>(p.gate)[(size_t)m * p.ldg + idx])));
          reinterpret_cast<T *>(p.out)[(size_t)m * n_out + idx] = DT<T>::from_f(o);
        }
      }
    }
  }
}
// the split form's last step: the key ranges' partial outputs are added in range order, gated and stored in D
template <typename T>
__global__ void __launch_bounds__(256) talk_attn_merge_kernel(const TalkAttn p) {
  const int m = blockIdx.x, n_out = p.heads * p.vdim, ns = p.nsplit;
  const float *part = p.part + (size_t)p.B * p.S * ns * p.heads * 2 + (size_t)m * ns * n_out;
  for (int idx = threadIdx.x; idx < n_out; idx += blockDim.x) {
    float o = 0.f;
    for (int s2 = 0; s2 < ns; s2++) o += part[(size_t)s2 * n_out + idx];
    if (p.gate) o *= 1.0f / (1.0f + expf(-DT<T>::to_f(reinterpret_cast<const T *>(p.gate)[(size_t)m * p.ldg + idx])));
    reinterpret_cast<T *>(p.out)[(size_t)m * n_out + idx] = DT<T>::from_f(o);
  }
}
int talk_attention(cudaStream_t st, int dtype, const TalkAttn &p, uint64_t *launches) {
  if (p.B < 1 || p.S < 1 || p.heads < 1 || p.kv_heads < 1 || p.heads % p.kv_heads || p.dim < 1 || p.vdim < 1 || (p.bias && p.bias_len < 1) || p.kv_heads > 64)
    return (int)cudaErrorInvalidValue;
  const int NT = 256;
  const size_t smem = ((size_t)p.heads * p.dim + 2 * p.heads + (size_t)p.heads * p.heads + 2 * (size_t)p.heads * NT) * sizeof(float);
  if (smem > 220 * 1024) return (int)cudaErrorInvalidValue;
  const int M = p.B * p.S;
  const bool split = p.part && p.nsplit > 1;
  MX_DISPATCH(dtype, {
    cudaError_t e = cudaSuccess;
    if (smem > 48 * 1024) {
      e = cudaFuncSetAttribute(talk_attn_kernel<T, 0>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (e == cudaSuccess) e = cudaFuncSetAttribute(talk_attn_kernel<T, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (e == cudaSuccess) e = cudaFuncSetAttribute(talk_attn_kernel<T, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (e != cudaSuccess) return (int)e;
    }
    if (!split) talk_attn_kernel<T, 0><<<M, NT, smem, st>>>(p);
    else {
      talk_attn_kernel<T, 1><<<dim3(M, p.nsplit), NT, smem, st>>>(p);
      talk_attn_kernel<T, 2><<<dim3(M, p.nsplit), NT, smem, st>>>(p);
      talk_attn_merge_kernel<T><<<M, 256, 0, st>>>(p);
    }
  });
  MX_DONE(split ? 3 : 1);
}

// ---- the matrix-product form: softmax + head mixing between the two products
// pass 1: a warp per (head, token) row: maximum and sum of exp over the keys the token sees
__global__ void __launch_bounds__(256) talk_softmax_stats_kernel(const TalkSoftmax p) {
  const long row = ((long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (row >= (long)p.heads * p.n_tok) return;
  const int h = (int)(row / p.n_tok), t = (int)(row % p.n_tok), pos = p.pos_first + t;
  const float *sr = p.scores + (size_t)row * p.kp;
  float mx = -INFINITY, l = 0.f;
  for (int j = lane; j <= pos; j += 32) {
    const float s = fmaf(sr[j], p.scale, p.bias ? p.bias[(size_t)min(pos - j, p.bias_len - 1) * p.heads + h] : 0.f);
    const float mn = fmaxf(mx, s);
    l = l * expf(mx - mn) + expf(s - mn);
    mx = mn;
  }
  const float m_all = warp_max(mx);
  l = warp_sum(mx > -INFINITY ? l * expf(mx - m_all) : 0.f);
  if (lane == 0) {
    p.stats[2 * row] = m_all;
    p.stats[2 * row + 1] = l;
  }
}
// pass 2 for up to HP heads: a CTA per token; a thread owns four adjacent keys: 16-byte reads of the scores, the normalised
// weights of all heads in registers, a row of the mixing matrix (read from shared memory four entries at a time) serves the four
// keys, and hi and lo leave as 8-byte stores
template <typename T, int HP>
__global__ void __launch_bounds__(256) talk_softmax_mix_regs_kernel(const TalkSoftmax p) {
  __shared__ __align__(16) float tk[HP * HP];
  __shared__ float M_[HP], L_[HP];
  const int H = p.heads, NT = blockDim.x, t = blockIdx.x, pos = p.pos_first + t;
  for (int i = threadIdx.x; i < HP * HP; i += NT) {
    const int hh = i / HP, g = i % HP;
    tk[i] = (hh < H && g < H) ? (p.talk ? DT<T>::to_f(reinterpret_cast<const T *>(p.talk)[hh * H + g]) : (hh == g ? 1.f : 0.f)) : 0.f;
  }
  for (int g = threadIdx.x; g < HP; g += NT) {
    M_[g] = g < H ? p.stats[2 * ((size_t)g * p.n_tok + t)] : 0.f;
    L_[g] = g < H ? 1.0f / p.stats[2 * ((size_t)g * p.n_tok + t) + 1] : 1.f;
  }
  __syncthreads();
  T *w = reinterpret_cast<T *>(p.w);
  for (int j0 = 4 * threadIdx.x; j0 < p.kp; j0 += 4 * NT) {
    float pr[HP][4];
    if (j0 > pos) {   // nothing of these four keys is seen: zeros
#pragma unroll 4
      for (int hh = 0; hh < H; hh++) {
        T *wr = w + ((size_t)hh * p.n_tok + t) * 2 * p.kp;
        *reinterpret_cast<uint2 *>(wr + j0) = make_uint2(0u, 0u);
        *reinterpret_cast<uint2 *>(wr + p.kp + j0) = make_uint2(0u, 0u);
      }
      continue;
    }
#pragma unroll
    for (int g = 0; g < HP; g++) {
      pr[g][0] = pr[g][1] = pr[g][2] = pr[g][3] = 0.f;
      if (g < H) {
        const float4 s4 = *reinterpret_cast<const float4 *>(p.scores + ((size_t)g * p.n_tok + t) * p.kp + j0);
        const float sv[4] = {s4.x, s4.y, s4.z, s4.w};
#pragma unroll
        for (int e = 0; e < 4; e++)
          if (j0 + e <= pos) {
            const float sc = fmaf(sv[e], p.scale, p.bias ? p.bias[(size_t)min(pos - j0 - e, p.bias_len - 1) * H + g] : 0.f);
            pr[g][e] = expf(sc - M_[g]) * L_[g];
          }
      }
    }
#pragma unroll 2
    for (int hh = 0; hh < H; hh++) {
      float v[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int g = 0; g < HP; g += 4) {
        const float4 t4 = *reinterpret_cast<const float4 *>(tk + hh * HP + g);
#pragma unroll
        for (int e = 0; e < 4; e++) {
          v[e] = fmaf(t4.x, pr[g][e], v[e]);
          v[e] = fmaf(t4.y, pr[g + 1][e], v[e]);
          v[e] = fmaf(t4.z, pr[g + 2][e], v[e]);
          v[e] = fmaf(t4.w, pr[g + 3][e], v[e]);
        }
      }
      typedef typename Bits16<T>::type B;
      float lo[4];
#pragma unroll
      for (int e = 0; e < 4; e++) lo[e] = v[e] - rnd<B>(v[e]);
      T *wr = w + ((size_t)hh * p.n_tok + t) * 2 * p.kp;
      *reinterpret_cast<uint2 *>(wr + j0) = make_uint2(pack2x<B>(v[0], v[1]), pack2x<B>(v[2], v[3]));
      *reinterpret_cast<uint2 *>(wr + p.kp + j0) = make_uint2(pack2x<B>(lo[0], lo[1]), pack2x<B>(lo[2], lo[3]));
    }
  }
}
// pass 2: a CTA per token: every thread normalises the scores of its keys for all heads, mixes them and stores hi | lo
template <typename T>
__global__ void __launch_bounds__(256) talk_softmax_mix_kernel(const TalkSoftmax p) {
  extern __shared__ float sm[];
  const int H = p.heads, NT = blockDim.x, t = blockIdx.x, pos = p.pos_first + t;
  float *M_ = sm, *L_ = M_ + H, *tk = L_ + H, *pg = tk + H * H;   // pg[g * NT + tid]
  for (int g = threadIdx.x; g < H; g += NT) {
    M_[g] = p.stats[2 * ((size_t)g * p.n_tok + t)];
    L_[g] = p.stats[2 * ((size_t)g * p.n_tok + t) + 1];
  }
  if (p.talk)
    for (int i = threadIdx.x; i < H * H; i += NT) tk[i] = DT<T>::to_f(reinterpret_cast<const T *>(p.talk)[i]);
  __syncthreads();
  T *w = reinterpret_cast<T *>(p.w);
  for (int j = threadIdx.x; j < p.kp; j += NT) {
    const bool seen = j <= pos;
    if (seen) {
      const int dist = min(pos - j, p.bias_len - 1);
      for (int g = 0; g < H; g++) {
        const float s = fmaf(p.scores[((size_t)g * p.n_tok + t) * p.kp + j], p.scale, p.bias ? p.bias[(size_t)dist * H + g] : 0.f);
        pg[g * NT + threadIdx.x] = expf(s - M_[g]) / L_[g];
      }
    }
    for (int hh = 0; hh < H; hh++) {
      float v = 0.f;
      if (seen) {
        if (p.talk)
          for (int g = 0; g < H; g++) v = fmaf(tk[hh * H + g], pg[g * NT + threadIdx.x], v);
        else v = pg[hh * NT + threadIdx.x];
      }
      const T hi = DT<T>::from_f(v);
      T *wr = w + ((size_t)hh * p.n_tok + t) * 2 * p.kp;
      wr[j] = hi;
      wr[p.kp + j] = DT<T>::from_f(v - DT<T>::to_f(hi));
    }
  }
}
int talk_softmax(cudaStream_t st, int dtype, const TalkSoftmax &p, uint64_t *launches) {
  if (p.n_tok < 1 || p.heads < 1 || p.kp < 1 || dtype == 2 || (p.bias && p.bias_len < 1)) return (int)cudaErrorInvalidValue;
  const long rows = (long)p.heads * p.n_tok;
  const size_t smem = ((size_t)2 * p.heads + (size_t)p.heads * p.heads + (size_t)p.heads * 256) * sizeof(float);
  if (smem > 200 * 1024) return (int)cudaErrorInvalidValue;
  talk_softmax_stats_kernel<<<(unsigned)((rows + 7) / 8), 256, 0, st>>>(p);
  MX_DISPATCH(dtype, {
    if (p.heads <= 4) talk_softmax_mix_regs_kernel<T, 4><<<p.n_tok, 256, 0, st>>>(p);
    else if (p.heads <= 8) talk_softmax_mix_regs_kernel<T, 8><<<p.n_tok, 256, 0, st>>>(p);
    else if (p.heads <= 16) talk_softmax_mix_regs_kernel<T, 16><<<p.n_tok, 256, 0, st>>>(p);
    else if (p.heads <= 32) talk_softmax_mix_regs_kernel<T, 32><<<p.n_tok, 256, 0, st>>>(p);
    else {
      if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(talk_softmax_mix_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
      }
      talk_softmax_mix_kernel<T><<<p.n_tok, 256, smem, st>>>(p);
    }
  });
  MX_DONE(2);
}
template <typename T>
__global__ void rows_by_head_kernel(const T *__restrict__ src, int ld, T *__restrict__ dst, int n_tok, int heads, int dim) {
  const int t = blockIdx.x;
  for (int i = threadIdx.x; i < heads * dim; i += blockDim.x) dst[((size_t)(i / dim) * n_tok + t) * dim + i % dim] = src[(size_t)t * ld + i];
}
int rows_by_head(cudaStream_t st, int dtype, const void *src, int ld, void *dst, int n_tok, int heads, int dim, uint64_t *launches) {
  MX_DISPATCH(dtype, (rows_by_head_kernel<T><<<n_tok, 256, 0, st>>>(reinterpret_cast<const T *>(src), ld, reinterpret_cast<T *>(dst), n_tok, heads, dim)));
  MX_DONE(1);
}
template <typename T>
__global__ void rows_to_tokens_kernel(const T *__restrict__ o, const T *__restrict__ gate, int ldg, T *__restrict__ out, int ldo, int n_tok, int heads, int vdim) {
  const int t = blockIdx.x;
  for (int i = threadIdx.x; i < heads * vdim; i += blockDim.x) {
    float v = DT<T>::to_f(o[((size_t)(i / vdim) * n_tok + t) * vdim + i % vdim]);
    if (gate) v *= 1.0f / (1.0f + expf(-DT<T>::to_f(gate[(size_t)t * ldg + i])));
    out[(size_t)t * ldo + i] = DT<T>::from_f(v);
  }
}
int rows_to_tokens(cudaStream_t st, int dtype, const void *o, const void *gate, int ldg, void *out, int ldo, int n_tok, int heads, int vdim,
                   uint64_t *launches) {
  MX_DISPATCH(dtype, (rows_to_tokens_kernel<T><<<n_tok, 256, 0, st>>>(reinterpret_cast<const T *>(o), reinterpret_cast<const T *>(gate), ldg,
                                                                       reinterpret_cast<T *>(out), ldo, n_tok, heads, vdim)));
  MX_DONE(1);
}
// a CTA transposes a tile of 32 tokens x 32 value entries through shared memory, so that reads and writes are both contiguous
template <typename T>
__global__ void values_transposed_kernel(const T *__restrict__ src, int ld, int col0, T *__restrict__ vt, int S, int kv_heads, int vdim, int cap_t, int pos0) {
  __shared__ T tile[32][33];
  const int b = blockIdx.z, t0 = blockIdx.x * 32, e0 = blockIdx.y * 32, n = kv_heads * vdim;
  for (int r = threadIdx.y; r < 32; r += blockDim.y) {
    const int t = t0 + r, e = e0 + threadIdx.x;
    if (t < S && e < n) tile[r][threadIdx.x] = src[((size_t)b * S + t) * ld + col0 + e];
  }
  __syncthreads();
  for (int r = threadIdx.y; r < 32; r += blockDim.y) {
    const int e = e0 + r, t = t0 + threadIdx.x;
    if (t < S && e < n) vt[((size_t)b * n + e) * cap_t + pos0 + t] = tile[threadIdx.x][r];
  }
}
int values_transposed_append(cudaStream_t st, int dtype, const void *src, int ld, int col0, void *vt, int B, int S, int kv_heads, int vdim, int cap_t,
                             int pos0, uint64_t *launches) {
  const dim3 grid((S + 31) / 32, (kv_heads * vdim + 31) / 32, B), block(32, 8);
  MX_DISPATCH(dtype, (values_transposed_kernel<T><<<grid, block, 0, st>>>(reinterpret_cast<const T *>(src), ld, col0, reinterpret_cast<T *>(vt), S, kv_heads,
                                                                          vdim, cap_t, pos0)));
  MX_DONE(1);
}

template <typename T>
__global__ void distance_bias_kernel(const T *__restrict__ rel, const int *__restrict__ bucket, float *__restrict__ bias, int len, int heads) {
  const int idx = blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= len * heads) return;
  bias[idx] = DT<T>::to_f(rel[(size_t)bucket[idx / heads] * heads + idx % heads]);
}
int distance_bias_table(cudaStream_t st, int dtype, const void *rel, const int *bucket, float *bias, int len, int heads, uint64_t *launches) {
  if (len < 1 || heads < 1) return (int)cudaErrorInvalidValue;
  MX_DISPATCH(dtype, (distance_bias_kernel<T><<<(len * heads + 255) / 256, 256, 0, st>>>(reinterpret_cast<const T *>(rel), bucket, bias, len, heads)));
  MX_DONE(1);
}

// ---------------------------------------------------------------------------------------------- embedding with tables
template <typename T>
__global__ void __launch_bounds__(128) embed_tables_kernel(const EmbedTables p) {
  const int r = blockIdx.x, b = r / p.S, t = r % p.S;
  uint32_t id = p.ids[r];
  if (id >= (uint32_t)p.vocab) id = 0;
  const T *E = reinterpret_cast<const T *>(p.E) + (size_t)id * p.W;
  const T *bg = nullptr, *ps = nullptr;
  if (p.bigram) {
    long long row = p.buckets;  // a sequence's first token
    if (t > 0 || p.pos0 > 0) {
      const long long prev = t > 0 ? p.ids[r - 1] : p.ids[(size_t)p.B * p.S + b];
      row = (prev * (long long)p.mul_prev + (long long)id * p.mul_cur) % p.buckets;
    }
    bg = reinterpret_cast<const T *>(p.bigram) + (size_t)row * p.W;
  }
  if (p.pos) ps = reinterpret_cast<const T *>(p.pos) + (size_t)(p.pos0 + t) * p.W;
  for (int i = threadIdx.x; i < p.W; i += blockDim.x) {
    float v = DT<T>::to_f(E[i]);
    if (p.scale != 0.f) v *= p.scale;
    if (bg) v += DT<T>::to_f(bg[i]);
    if (ps) v += DT<T>::to_f(ps[i]);
    p.x[(size_t)r * p.W + i] = v;
  }
}
int embed_tables(cudaStream_t st, int dtype, const EmbedTables &p, uint64_t *launches) {
  if (p.B < 1 || p.S < 1 || (p.bigram && p.buckets < 1)) return (int)cudaErrorInvalidValue;
  MX_DISPATCH(dtype, (embed_tables_kernel<T><<<p.B * p.S, 128, 0, st>>>(p)));
  MX_DONE(1);
}

// ---------------------------------------------------------------------------------------------- stream injection
template <typename T>
__global__ void __launch_bounds__(256) stream_inject_kernel(float *x, const float *x0, const T *vec, int W) {
  const size_t m = blockIdx.x;
  for (int i = threadIdx.x; i < W; i += blockDim.x) {
    float v = x[m * W + i];
    if (x0) v += x0[m * W + i];
    x[m * W + i] = v + DT<T>::to_f(vec[i]);
  }
}
int stream_inject(cudaStream_t st, int dtype, float *x, const float *x0, const void *vec, int M, int W, uint64_t *launches) {
  MX_DISPATCH(dtype, (stream_inject_kernel<T><<<M, 256, 0, st>>>(x, x0, reinterpret_cast<const T *>(vec), W)));
  MX_DONE(1);
}

}  // namespace mx
}  // namespace cake
