// f32_stream.cuh — the pieces of a block whose residual stream is FP32 (layer-list models, cake_b200_block_load_spec):
//
//   embed_f32_kernel         x[t] = float(E[id[t]])
//   norm_shift_rows_kernel   RMS norm in fp32 with a scalar or a vector gain, and the token shift
//                            hs = h + (h_prev - h) * shift  (h_prev = the previous position's h, zeros at position 0);
//                            the operands of the matrix products leave in D
//   gemm_rows_kernel         C = A[M,K] · W[N,K]^T on the CUDA cores, fp32 accumulation, with the epilogues this block needs:
//                            store in D | act(gate) * up on row-interleaved gate/up | fp32 residual add | soft-capped fp32
//                            logits.  It serves every shape and D = float (true fp32: one FFMA per product, no TF32); the
//                            tcgen05 GEMM (gemm_tc.cuh) takes over for 16-bit D at the shapes its tiles cover.
//   rows_to_cache_kernel     appends a column range of a row-major activation to a [batch, kv_heads, cap, head_dim] cache
//
// Nothing here follows a reference file: the reference has no block with an fp32 residual stream.
#pragma once
#include "common.cuh"

namespace cake {

// ---- embedding gather into the fp32 stream ------------------------------------------------------------------------------
template <typename T> struct EmbedBits { typedef T type; };
template <> struct EmbedBits<float> { typedef __nv_bfloat16 type; };  // never taken for float (sizeof test); keeps unpack8 instantiable
template <typename T>
__global__ void embed_f32_kernel(const T *__restrict__ E, const uint32_t *__restrict__ ids, float *__restrict__ x, int n_tok,
                                 int H, int vocab, float scale /* 0 = none */) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  if (t >= n_tok) return;
  uint32_t id = ids[t];
  if (id >= (uint32_t)vocab) id = 0;
  const T *src = E + (size_t)id * H;
  float *dst = x + (size_t)t * H;
  if (sizeof(T) == 2 && (H & 7) == 0 && scale == 0.f) {  // 16-byte loads, two 16-byte stores per thread and step
    const uint4 *s4 = reinterpret_cast<const uint4 *>(src);
    float4 *d4 = reinterpret_cast<float4 *>(dst);
    for (int i = threadIdx.x; i < H / 8; i += blockDim.x) {
      float f[8];
      unpack8<typename EmbedBits<T>::type>(s4[i], f);
      d4[2 * i] = make_float4(f[0], f[1], f[2], f[3]);
      d4[2 * i + 1] = make_float4(f[4], f[5], f[6], f[7]);
    }
    return;
  }
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    const float v = DT<T>::to_f(src[i]);
    dst[i] = scale == 0.f ? v : v * scale;
  }
}

// ---- RMS norm (scalar or vector gain) + token shift ---------------------------------------------------------------------
// One CTA per output row r.  Source row = rows ? rows[r] : r of x [.., n] (fp32).  With S > 0 the rows are (b, t) pairs of
// a [B, S, n] step that starts at absolute position pos0, and the shifted copy hs is produced from the previous row's h:
//   t > 0            the row before, normalised again here (reading it twice is cheaper than a second kernel)
//   t == 0, pos0 > 0 state_in[b] — the last h of the previous call, kept in fp32
//   t == 0, pos0 == 0 zeros
// The last row of every b leaves its h in state_out[b] (a different buffer than state_in: other CTAs still read that).
template <typename T> __device__ __forceinline__ void store4(T *dst, float a, float b, float c, float d) {
  *reinterpret_cast<uint2 *>(dst) = make_uint2(pack2x<T>(a, b), pack2x<T>(c, d));
}
template <> __device__ __forceinline__ void store4<float>(float *dst, float a, float b, float c, float d) {
  *reinterpret_cast<float4 *>(dst) = make_float4(a, b, c, d);
}

// Source row of output row r: rows ? rows[r] : r * row_mul + row_add (the last position of every batch row needs no table).
template <typename T>
__global__ void __launch_bounds__(256) norm_shift_rows_kernel(const float *__restrict__ x, const int *__restrict__ rows, int row_mul, int row_add,
                                                              const T *__restrict__ g, int g_stride,
                                                              const T *__restrict__ shift, const float *__restrict__ state_in,
                                                              float *__restrict__ state_out, T *__restrict__ h_out,
                                                              T *__restrict__ hs_out, int S, int n, float eps, int pos0,
                                                              float g_add /* gain = g + g_add: gains stored as offsets */) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float red[2][8];
  const int r = blockIdx.x;
  const size_t src = rows ? (size_t)rows[r] : (size_t)r * row_mul + row_add;
  const float *xr = x + src * n;
  const bool shifted = shift != nullptr;
  const int t = shifted ? r % S : 0, b = shifted ? r / S : 0;
  const bool prev_row = shifted && t > 0;
  const float *xp = xr - n;
  const bool vec = (n & 3) == 0;   // rows of 16-byte multiples: 16-byte loads, 8- / 16-byte stores
  float ss = 0.f, sp = 0.f;
  if (vec) {
    const float4 *x4 = reinterpret_cast<const float4 *>(xr), *p4 = reinterpret_cast<const float4 *>(xp);
    for (int i = threadIdx.x; i < n / 4; i += blockDim.x) {
      const float4 v = x4[i];
      ss = fmaf(v.x, v.x, ss); ss = fmaf(v.y, v.y, ss); ss = fmaf(v.z, v.z, ss); ss = fmaf(v.w, v.w, ss);
      if (prev_row) {
        const float4 u = p4[i];
        sp = fmaf(u.x, u.x, sp); sp = fmaf(u.y, u.y, sp); sp = fmaf(u.z, u.z, sp); sp = fmaf(u.w, u.w, sp);
      }
    }
  } else {
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
      const float v = xr[i];
      ss = fmaf(v, v, ss);
      if (prev_row) {
        const float u = xp[i];
        sp = fmaf(u, u, sp);
      }
    }
  }
  ss = warp_sum(ss);
  sp = warp_sum(sp);
  if ((threadIdx.x & 31) == 0) { red[0][threadIdx.x >> 5] = ss; red[1][threadIdx.x >> 5] = sp; }
  __syncthreads();
  float tot = 0.f, totp = 0.f;
  for (int i = 0; i < (int)(blockDim.x >> 5); i++) { tot += red[0][i]; totp += red[1][i]; }
  const float inv = 1.0f / sqrtf(tot / (float)n + eps);
  const float invp = 1.0f / sqrtf(totp / (float)n + eps);
  const bool from_state = shifted && t == 0 && pos0 > 0;
  const bool last = shifted && t == S - 1;
  if (vec) {  // the second read of the row comes out of L1 / L2
    const float4 *x4 = reinterpret_cast<const float4 *>(xr), *p4 = reinterpret_cast<const float4 *>(xp);
    const float4 *s4 = reinterpret_cast<const float4 *>(state_in + (from_state ? (size_t)b * n : 0));
    for (int i = threadIdx.x; i < n / 4; i += blockDim.x) {
      const float4 v = x4[i];
      float gi[4], h[4];
#pragma unroll
      for (int e = 0; e < 4; e++) gi[e] = DT<T>::to_f(g[(size_t)(4 * i + e) * g_stride]) + g_add;
      h[0] = v.x * inv * gi[0]; h[1] = v.y * inv * gi[1]; h[2] = v.z * inv * gi[2]; h[3] = v.w * inv * gi[3];
      if (h_out) store4<T>(h_out + (size_t)r * n + 4 * i, h[0], h[1], h[2], h[3]);
      if (shifted) {
        float hp[4] = {0.f, 0.f, 0.f, 0.f};
        if (prev_row) {
          const float4 u = p4[i];
          hp[0] = u.x * invp * gi[0]; hp[1] = u.y * invp * gi[1]; hp[2] = u.z * invp * gi[2]; hp[3] = u.w * invp * gi[3];
        } else if (from_state) {
          const float4 u = s4[i];
          hp[0] = u.x; hp[1] = u.y; hp[2] = u.z; hp[3] = u.w;
        }
        float o[4];
#pragma unroll
        for (int e = 0; e < 4; e++) o[e] = h[e] + (hp[e] - h[e]) * DT<T>::to_f(shift[4 * i + e]);
        store4<T>(hs_out + (size_t)r * n + 4 * i, o[0], o[1], o[2], o[3]);
        if (last) *reinterpret_cast<float4 *>(state_out + (size_t)b * n + 4 * i) = make_float4(h[0], h[1], h[2], h[3]);
      }
    }
    return;
  }
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const float gi = DT<T>::to_f(g[(size_t)i * g_stride]) + g_add;
    const float h = xr[i] * inv * gi;
    if (h_out) h_out[(size_t)r * n + i] = DT<T>::from_f(h);
    if (shifted) {
      const float hp = prev_row ? xp[i] * invp * gi : (from_state ? state_in[(size_t)b * n + i] : 0.f);
      hs_out[(size_t)r * n + i] = DT<T>::from_f(h + (hp - h) * DT<T>::to_f(shift[i]));
      if (last) state_out[(size_t)b * n + i] = h;
    }
  }
}

// ---- generic GEMM with the fp32-stream epilogues --------------------------------------------------------------------------
enum { RE_STORE = 0, RE_GATE_UP = 1, RE_RESIDUAL_F32 = 2, RE_SOFTCAP_F32 = 3 };
struct RowsGemm {
  const void *A;    // [M, lda] D
  const void *W;    // [N, K] D
  const float *R;   // RE_RESIDUAL_F32: [M, N] fp32
  void *C;          // RE_STORE: [M, ldc] D;  RE_GATE_UP: [M, ldc] D, N/2 columns written;  else [M, N] fp32
  int M, N, K, lda, ldc;
  int act;          // RE_GATE_UP: 0 silu, 1 tanh-gelu, 2 clamped (gated_pair; the limit travels in cap)
  float cap;        // RE_SOFTCAP_F32: 0 = none
  const float *rs = nullptr;  // RE_RESIDUAL_F32: optional [M] fp32, C = R + rs[m] * (A W^T) (a per-row gate on the product)
  const void *bias = nullptr; // RE_STORE: optional [N] D added to the fp32 sum before it is rounded
};
constexpr int RG_BM = 64, RG_BN = 64, RG_BK = 16;
template <typename T, int EPI>
__global__ void __launch_bounds__(256) gemm_rows_kernel(const RowsGemm p) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float As[RG_BK][RG_BM + 4];
  __shared__ float Ws[RG_BK][RG_BN + 4];
  const T *A = reinterpret_cast<const T *>(p.A);
  const T *W = reinterpret_cast<const T *>(p.W);
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  const int m0 = blockIdx.y * RG_BM, n0 = blockIdx.x * RG_BN;
  float acc[4][4] = {};
  for (int k0 = 0; k0 < p.K; k0 += RG_BK) {
    for (int i = threadIdx.x; i < RG_BM * RG_BK; i += 256) {
      const int r = i / RG_BK, c = i % RG_BK;
      As[c][r] = (m0 + r < p.M && k0 + c < p.K) ? DT<T>::to_f(A[(size_t)(m0 + r) * p.lda + k0 + c]) : 0.f;
      Ws[c][r] = (n0 + r < p.N && k0 + c < p.K) ? DT<T>::to_f(W[(size_t)(n0 + r) * p.K + k0 + c]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < RG_BK; k++) {
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
    if (EPI == RE_GATE_UP) {  // columns (2c, 2c+1) of this thread = (gate_c, up_c)
      T *C = reinterpret_cast<T *>(p.C);
#pragma unroll
      for (int j = 0; j < 4; j += 2) {
        const int n = n0 + tx * 4 + j;
        if (n + 1 < p.N) C[(size_t)m * p.ldc + n / 2] = DT<T>::from_f(gated_pair<T>(acc[i][j], acc[i][j + 1], p.act, p.cap));
      }
    } else {
#pragma unroll
      for (int j = 0; j < 4; j++) {
        const int n = n0 + tx * 4 + j;
        if (n >= p.N) continue;
        if (EPI == RE_STORE) reinterpret_cast<T *>(p.C)[(size_t)m * p.ldc + n] = DT<T>::from_f(p.bias ? acc[i][j] + DT<T>::to_f(reinterpret_cast<const T *>(p.bias)[n]) : acc[i][j]);
        else if (EPI == RE_RESIDUAL_F32) reinterpret_cast<float *>(p.C)[(size_t)m * p.N + n] = p.R[(size_t)m * p.N + n] + (p.rs ? p.rs[m] * acc[i][j] : acc[i][j]);
        else reinterpret_cast<float *>(p.C)[(size_t)m * p.N + n] = p.cap > 0.f ? p.cap * tanhf(acc[i][j] / p.cap) : acc[i][j];
      }
    }
  }
}

// ---- append a column range of an activation to a [B, n_kv, cap, hd] cache -------------------------------------------------
// src row (b, t) = src[(b*S + t) * ld + col0 ..], n_kv * hd values; destination row pos0 + t of every kv head.
template <typename T>
__global__ void rows_to_cache_kernel(const T *__restrict__ src, T *__restrict__ cache, int S, int ld, int col0, int n_kv, int hd,
                                     int cap, int pos0) {
  pdl_launch_dependents();
  pdl_wait();
  const int r = blockIdx.x, b = r / S, t = r % S;
  const T *s = src + (size_t)r * ld + col0;
  constexpr int VE = 16 / (int)sizeof(T);  // elements per 16-byte copy
  if (hd % VE == 0 && ld % VE == 0 && col0 % VE == 0) {
    const int cpr = hd / VE;  // 16-byte chunks per head row
    for (int i = threadIdx.x; i < n_kv * cpr; i += blockDim.x) {
      const int g = i / cpr, c = i % cpr;
      reinterpret_cast<uint4 *>(cache + (((size_t)b * n_kv + g) * cap + pos0 + t) * hd)[c] = reinterpret_cast<const uint4 *>(s + (size_t)g * hd)[c];
    }
    return;
  }
  for (int i = threadIdx.x; i < n_kv * hd; i += blockDim.x) {
    const int g = i / hd, d = i % hd;
    cache[(((size_t)b * n_kv + g) * cap + pos0 + t) * hd + d] = s[i];
  }
}

// ---- fp32 logits -> the 16-bit dtype the samplers read --------------------------------------------------------------------
template <typename T>
__global__ void f32_to_T_kernel(const float *__restrict__ src, T *__restrict__ dst, size_t n) {
  pdl_launch_dependents();
  pdl_wait();
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) dst[i] = DT<T>::from_f(src[i]);
}

}  // namespace cake
