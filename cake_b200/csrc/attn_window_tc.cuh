// attn_window_tc.cuh — the windowed, soft-capped, distance-biased attention of attn_window_bias.cuh for prompt portions with
// head_dim 128 in 16-bit D, on the 5th-generation tensor cores: attn_prefill_tc_kernel (attn_prefill_tc.cuh) with
//   * the tile loop starting at the first tile the window of the CTA's first row reaches,
//   * the score modifiers applied by the softmax warps before the mask (the modified score is in natural units, so the
//     exponent constant is log2 e), rows that see nothing in a tile keeping a -inf reference,
//   * the K tensor map given twice: the keys double as values, the V ring is filled from the same cache rows,
//   * the head gate and the caller's row stride in the epilogue,
//   * optionally: the tiles of the kept first keys ahead of the window's tiles, a sink logit in the denominator, a gate per head
//     or per output element from a buffer of its own, and key / value buffers whose first row is a later position (key0).
// Warp roles, barriers, TMEM layout and the P_hi + P_lo operand are those of attn_prefill_tc_kernel; see there.
// Cost model: four MUFU operations per score (tanh = ex2 + rcp, ln, the softmax's ex2) against one in the plain kernel make
// the softmax warps, not the MMAs, the bound of this kernel.
#pragma once
#include "attn_prefill_tc.cuh"
#include "attn_window_bias.cuh"

namespace cake {

template <typename T>
__global__ void __launch_bounds__(FT_THREADS, 2)
attn_window_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                      const __grid_constant__ CUtensorMap map_v, const WinAttn p, float tau_log2) {
  const int S = p.S, n_heads = p.heads, n_kv = p.n_kv, pos0 = p.pos0;
  constexpr float scale_log2 = 1.4426950408889634f;  // the modified score is in natural units: p = 2^((s - m) log2 e)
  extern __shared__ unsigned char ft_smem_raw[];
  unsigned char *smem = reinterpret_cast<unsigned char *>((reinterpret_cast<uintptr_t>(ft_smem_raw) + 1023) & ~(uintptr_t)1023);
  unsigned char *q_s = smem;
  unsigned char *k_s = q_s + FT_Q_BYTES;       // [2] stages
  unsigned char *v_s = k_s + 2 * FT_KV_BYTES;  // [2] stages
  uint64_t *bars = reinterpret_cast<uint64_t *>(v_s + 2 * FT_KV_BYTES);
  uint64_t *q_full = bars, *k_full = bars + 1, *k_empty = bars + 3, *v_full = bars + 5, *v_empty = bars + 7, *s_full = bars + 9,
           *p_full = bars + 11, *o_full = bars + 12;
  uint32_t *tmem_ptr = reinterpret_cast<uint32_t *>(bars + 13);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int mt = gridDim.x - 1 - blockIdx.x;  // heavy (late) query tiles first
  const int h = blockIdx.y, b = blockIdx.z, kvh = h / (n_heads / n_kv);
  const int m0 = mt * FT_BM;
  const int kv_end = pos0 + min(S, m0 + FT_BM);  // keys visible to the last query of this tile
  // tiles [j_lo, j_end): from the one that holds the first key the tile's first row sees; rings and phases count from j_lo
  const int j_lo = p.window > 0 ? max(0, pos0 + m0 - p.window + 1) / FT_BN : 0;
  // kept first keys that lie before the window's first tile come first: iteration j works on key tile j (j < n_kept) or
  // j_lo + j - n_kept
  const int n_kept = min(j_lo, (p.keep_first + FT_BN - 1) / FT_BN);
  const int n_tiles = n_kept + (kv_end + FT_BN - 1) / FT_BN - j_lo;
  const int j_add = j_lo - n_kept;

  if (threadIdx.x == 0) {
    for (int i = 0; i < 13; i++) mbar_init(&bars[i], i == 11 ? 128u : 1u);
    mbar_fence_init();
  }
  if (warp == 5) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_ptr)), "n"(FT_TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  pdl_launch_dependents();
  pdl_wait();
  const uint32_t tmem_base = *tmem_ptr;
  const uint32_t tmem_o = tmem_base + 128u;  // S/P buffer i at columns 64 i

  if (warp == 4) {
    // ===================== TMA producer ====================================================================
    if (lane == 0) {
      asm volatile("prefetch.tensormap [%0];" ::"l"(&map_q) : "memory");
      asm volatile("prefetch.tensormap [%0];" ::"l"(&map_k) : "memory");
      asm volatile("prefetch.tensormap [%0];" ::"l"(&map_v) : "memory");
      mbar_arrive_expect_tx(q_full, FT_Q_BYTES);
      tma_load_3d(q_s, &map_q, h * FT_HD, m0, b, q_full);
      tma_load_3d(q_s + FT_Q_BYTES / 2, &map_q, h * FT_HD + 64, m0, b, q_full);
      const int slab = b * n_kv + kvh;
      for (int j = 0; j < n_tiles; j++) {
        const int st = j & 1;
        const uint32_t eph = (uint32_t)((j >> 1) - 1) & 1u;  // the stage's previous use (tile j-2) has been consumed
        unsigned char *kd = k_s + st * FT_KV_BYTES, *vd = v_s + st * FT_KV_BYTES;
        if (j >= 2) mbar_wait(&k_empty[st], eph);
        mbar_arrive_expect_tx(&k_full[st], FT_KV_BYTES);
        const int krow = (j < n_kept ? j : j + j_add) * FT_BN - p.key0;  // rows before the buffer read as zeros and are masked
        tma_load_3d(kd, &map_k, 0, krow, slab, &k_full[st]);
        tma_load_3d(kd + FT_KV_BYTES / 2, &map_k, 64, krow, slab, &k_full[st]);
        if (j >= 2) mbar_wait(&v_empty[st], eph);
        mbar_arrive_expect_tx(&v_full[st], FT_KV_BYTES);
        tma_load_3d(vd, &map_v, 0, krow, slab, &v_full[st]);
        tma_load_3d(vd + FT_KV_BYTES / 2, &map_v, 64, krow, slab, &v_full[st]);
      }
    }
  } else if (warp == 5) {
    // ===================== MMA issuer (one thread) =========================================================
    if (lane == 0) {
      const uint32_t idesc_s = tc_idesc<T>(FT_BN);                   // M128 N64, A and B K-major
      const uint32_t idesc_o = tc_idesc<T>(FT_HD) | (1u << 16);      // M128 N128, A from TMEM, B (V) MN-major
      auto issue_s = [&](int j) {  // S_j = Q K_j^T into S buffer j&1
        const int st = j & 1;
        mbar_wait(&k_full[st], (uint32_t)(j >> 1) & 1u);
        tc_fence_after();
        const unsigned char *kt = k_s + st * FT_KV_BYTES;
#pragma unroll
        for (int k = 0; k < FT_HD / 16; k++) {  // head dims 16k..16k+15: box k/4, 32-byte slab k%4 inside the swizzle row
          const uint64_t da = tc_smem_desc(q_s + (k >> 2) * (FT_Q_BYTES / 2)) + (uint64_t)((k & 3) * 2);
          const uint64_t db = tc_smem_desc(kt + (k >> 2) * (FT_KV_BYTES / 2)) + (uint64_t)((k & 3) * 2);
          tc_mma_f16(tmem_base + (uint32_t)(st * 64), da, db, idesc_s, k ? 1u : 0u);
        }
        tc_commit(&k_empty[st]);
        tc_commit(&s_full[st]);
      };
      mbar_wait(q_full, 0);
      issue_s(0);
      for (int j = 0; j < n_tiles; j++) {
        const int st = j & 1;
        // S of the next tile first: its buffer held P of tile j-1, whose P V is already queued ahead of it in the pipe
        if (j + 1 < n_tiles) issue_s(j + 1);
        mbar_wait(p_full, (uint32_t)j & 1u);  // P_j in TMEM (over S_j), O rescaled
        mbar_wait(&v_full[st], (uint32_t)(j >> 1) & 1u);
        tc_fence_after();
        const unsigned char *vt = v_s + st * FT_KV_BYTES;
#pragma unroll
        for (int half = 0; half < 2; half++)
#pragma unroll
          for (int ks = 0; ks < FT_BN / 16; ks++) {  // keys 16ks..16ks+15 = 8 packed columns of P_hi (0..31) or P_lo (32..63)
            const uint32_t ta = tmem_base + (uint32_t)(st * 64 + half * 32 + ks * 8);
            const uint64_t db = ft_desc_mn(vt + ks * 2048, FT_KV_BYTES / 2);
            tc_mma_f16_ts(tmem_o, ta, db, idesc_o, (j | half | ks) ? 1u : 0u);
          }
        tc_commit(&v_empty[st]);
        tc_commit(o_full);
      }
    }
  } else {
    // ===================== softmax / correction / epilogue (thread = query row) =============================
    const int row = warp * 32 + lane;
    const int qp = pos0 + m0 + row;  // absolute position of this row's query
    const uint32_t lane_addr = (uint32_t)(warp * 32) << 16;
    float m_run = -INFINITY, l_run = 0.f;  // m_run: reference max of the modified scores
    const bool biased = p.r1 != nullptr;
    const float r1 = biased ? DT<T>::to_f(reinterpret_cast<const T *>(p.r1)[h]) : 0.f;
    const float r2 = biased ? DT<T>::to_f(reinterpret_cast<const T *>(p.r2)[h]) : 0.f;
    const float inv_cap2 = p.softcap > 0.f ? 2.0f / p.softcap : 0.f;
    for (int j = 0; j < n_tiles; j++) {
      const uint32_t tmem_sp = tmem_base + lane_addr + (uint32_t)((j & 1) * 64);
      mbar_wait(&s_full[j & 1], (uint32_t)(j >> 1) & 1u);
      tc_fence_after();
      float sv[FT_BN];
      {
        uint32_t r[32];
        tc_ld32(tmem_sp, r);
#pragma unroll
        for (int i = 0; i < 32; i++) sv[i] = __uint_as_float(r[i]);
        tc_ld32(tmem_sp + 32u, r);
#pragma unroll
        for (int i = 0; i < 32; i++) sv[32 + i] = __uint_as_float(r[i]);
      }
      // soft cap, distance bias, window: every score of the tile (the transcendentals dominate, a tile-level test would not pay)
      // Branch-free, so that the 64 independent chains of a row interleave (MUFU latency is what a softmax warp waits for):
      // the distance is carried as a float (exact below 2^24, no I2F on the MUFU pipe), masked entries take the arithmetic
      // with a clamped distance and are replaced by -inf at the end.
      float mx = -INFINITY;
      const float fd0 = (float)(qp - (j < n_kept ? j : j + j_add) * FT_BN);  // distance to the tile's first key
      const float fwin = p.window > 0 ? (float)p.window : 3.0e38f;
      const float fkept = (float)(qp - p.keep_first);  // key < keep_first  <=>  distance > qp - keep_first
#pragma unroll
      for (int i = 0; i < FT_BN; i++) {
        const float fd = fd0 - (float)i;
        float v = sv[i] * p.scale;
        if (p.softcap > 0.f) v = p.softcap * (1.0f - __fdividef(2.0f, __expf(v * inv_cap2) + 1.0f));
        if (biased) v -= r1 * __logf(fmaf(r2, fmaxf(fd, 0.f), 1.0f));
        v = (fd >= 0.f && (fd < fwin || fd > fkept)) ? v : -INFINITY;
        sv[i] = v;
        mx = fmaxf(mx, v);
      }
      // running max with lazy update: keep the old reference while the new max exceeds it by at most tau.  A row may see
      // nothing in a tile (its window starts later, or ended earlier): its reference stays -inf until a key shows up
      float fac = 1.f;
      bool resc = false;
      if ((mx - m_run) * scale_log2 > tau_log2) {
        fac = (m_run == -INFINITY) ? 0.f : ft_ex2((m_run - mx) * scale_log2);
        m_run = mx;
        resc = true;
      }
      // p = exp(s - m) = 2^(s c - m c), c = log2 e: one FFMA + one MUFU.EX2 per score; 2^-inf = 0 masks
      const float mc = (m_run == -INFINITY) ? 0.f : m_run * scale_log2;
      float rs = 0.f;
#pragma unroll
      for (int i = 0; i < FT_BN; i++) {
        const float pe = ft_ex2(fmaf(sv[i], scale_log2, -mc));
        sv[i] = pe;
        rs += pe;
      }
      l_run = l_run * fac + rs;
      if (j > 0) {
        mbar_wait(o_full, (uint32_t)(j - 1) & 1u);  // P V of the previous tile is complete: O stable
        tc_fence_after();
        if (__any_sync(0xffffffffu, resc)) {
#pragma unroll 1
          for (int c0 = 0; c0 < FT_HD; c0 += 32) {
            uint32_t r[32];
            tc_ld32(tmem_o + lane_addr + (uint32_t)c0, r);
#pragma unroll
            for (int i = 0; i < 32; i++) r[i] = __float_as_uint(__uint_as_float(r[i]) * fac);
            tc_st32(tmem_o + lane_addr + (uint32_t)c0, r);
          }
        }
      }
      // P = P_hi + P_lo, both in D, packed two keys per column over the S tile: columns 0..31 P_hi, 32..63 P_lo
      {
        uint32_t hi[32], lo[32];
#pragma unroll
        for (int i = 0; i < 32; i++) {
          const float p0 = sv[2 * i], p1 = sv[2 * i + 1];
          hi[i] = pack2x<T>(p0, p1);
          const float2 hf = DT<T>::unpack2(hi[i]);
          lo[i] = pack2x<T>(p0 - hf.x, p1 - hf.y);
        }
        tc_st32(tmem_sp, hi);
        tc_st32(tmem_sp + 32u, lo);
      }
      tc_wait_st();
      tc_fence_before();
      mbar_arrive(p_full);
    }
    // ---- epilogue: O / l, one rounding to D (attention.rs:346), store (b, s, h, hd) ---------------------------
    mbar_wait(o_full, (uint32_t)(n_tiles - 1) & 1u);
    tc_fence_after();
    const int t = m0 + row;
    float gate = 1.0f;
    const T *gsrc = reinterpret_cast<const T *>(p.gate) + (size_t)(b * S + t) * p.ldg;
    if (p.gate_mode == 1) {
      if (t < S) gate = 1.0f / (1.0f + expf(-DT<T>::to_f(gsrc[h])));
    } else if (p.gate_mode == 0 && p.gate_col >= 0 && t < S)
      gate = 1.0f / (1.0f + expf(-DT<T>::to_f(reinterpret_cast<const T *>(p.qkg)[(size_t)(b * S + t) * p.ld + p.gate_col + h])));
    // the sink counts once in the denominator, relative to the row's reference maximum (which holds at least the row's own key)
    if (p.sink) l_run += expf(DT<T>::to_f(reinterpret_cast<const T *>(p.sink)[h]) - m_run);
    const float inv = gate / l_run;
    T *dst = reinterpret_cast<T *>(p.y) + (size_t)(b * S + t) * p.ldy + h * FT_HD;
#pragma unroll 1
    for (int c0 = 0; c0 < FT_HD; c0 += 32) {
      uint32_t r[32];
      tc_ld32(tmem_o + lane_addr + (uint32_t)c0, r);
      if (t < S) {
        if (p.gate_mode == 2) {  // a gate per output element: 64 bytes of logits per 32 columns (ldg % 8 == 0, 16-byte base)
          const uint4 *g4 = reinterpret_cast<const uint4 *>(gsrc + h * FT_HD + c0);
#pragma unroll
          for (int q = 0; q < 4; q++) {
            const uint4 gv = g4[q];
            const uint32_t gw[4] = {gv.x, gv.y, gv.z, gv.w};
#pragma unroll
            for (int e = 0; e < 4; e++) {
              const float2 gl = DT<T>::unpack2(gw[e]);
              const int i = 8 * q + 2 * e;
              r[i] = __float_as_uint(__uint_as_float(r[i]) / (1.0f + expf(-gl.x)));
              r[i + 1] = __float_as_uint(__uint_as_float(r[i + 1]) / (1.0f + expf(-gl.y)));
            }
          }
        }
        uint32_t o[16];
#pragma unroll
        for (int i = 0; i < 16; i++) o[i] = pack2x<T>(__uint_as_float(r[2 * i]) * inv, __uint_as_float(r[2 * i + 1]) * inv);
        uint4 *d4 = reinterpret_cast<uint4 *>(dst + c0);
#pragma unroll
        for (int i = 0; i < 4; i++) d4[i] = make_uint4(o[4 * i], o[4 * i + 1], o[4 * i + 2], o[4 * i + 3]);
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 5) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "n"(FT_TMEM_COLS) : "memory");
  }
}

}  // namespace cake
