// cake_b200.cu — C ABI of libcake_b200.so (see include/cake_b200.h for the contract and the
// reference interfaces each entry replaces).  Host-side logic only: handles, buffers, kernel plans,
// the CUDA graph of the decode step and the NCCL p2p hand-off.  All math is in the .cuh kernels.
#include <cuda_runtime.h>
#include <dlfcn.h>
#include <math.h>
#include <nccl.h>
#include <stdarg.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <atomic>
#include <algorithm>
#include <chrono>
#include <mutex>
#include <thread>
#include <set>
#include <string>
#include <vector>

#include "../../include/cake_b200.h"
#include "attn_decode.cuh"
#include "attn_prefill.cuh"
#include "attn_prefill_tc.cuh"
#include "attn_window_bias.cuh"
#include "attn_window_tc.cuh"
#include "common.cuh"
#include "decode_mega.cuh"
#include "f32_stream.cuh"
#include "mixers.cuh"
#include "gemm_tc.cuh"
#include "gemv.cuh"
#include "prefill.cuh"
#include "sample.cuh"

using namespace cake;
typedef __nv_bfloat16 bf16;

// ------------------------------------------------------------------------------------------ errors
static thread_local char g_err[512] = "";
static int fail(int code, const char *fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}
#define CU(call)                                                                                              \
  do {                                                                                                        \
    cudaError_t e_ = (call);                                                                                  \
    if (e_ != cudaSuccess) return fail(CAKE_B200_ECUDA, "%s:%d %s -> %s", __FILE__, __LINE__, #call, cudaGetErrorString(e_)); \
  } while (0)
#define RC(call)              \
  do {                        \
    int rc_ = (call);         \
    if (rc_ != CAKE_B200_OK) return rc_; \
  } while (0)

struct cake_b200_ctx;
static int wait_loads(cake_b200_ctx *c);
extern "C" const char *cake_b200_last_error(void) { return g_err; }
extern "C" const char *cake_b200_version(void) { return "cake_b200 0.1 (sm_100a)"; }

// ------------------------------------------------------------------------------------------ NCCL (dlopen, like the reference's rocm/ffi.rs function table)
struct NcclApi {
  void *lib = nullptr;
  ncclResult_t (*GetUniqueId)(ncclUniqueId *) = nullptr;
  ncclResult_t (*CommInitRank)(ncclComm_t *, int, ncclUniqueId, int) = nullptr;
  ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
  ncclResult_t (*Send)(const void *, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t) = nullptr;
  ncclResult_t (*Recv)(void *, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t) = nullptr;
  const char *(*GetErrorString)(ncclResult_t) = nullptr;
  ncclResult_t (*GroupStart)() = nullptr;
  ncclResult_t (*GroupEnd)() = nullptr;
};
static NcclApi g_nccl;
static int nccl_load() {
  if (g_nccl.lib) return CAKE_B200_OK;
  const char *names[] = {getenv("CAKE_B200_NCCL_LIB"), "libnccl.so.2", "libnccl.so"};
  void *h = nullptr;
  for (const char *n : names) {
    if (!n) continue;
    h = dlopen(n, RTLD_NOW | RTLD_GLOBAL);
    if (h) break;
  }
  if (!h) return fail(CAKE_B200_ENCCL, "cannot dlopen libnccl.so.2 (set CAKE_B200_NCCL_LIB): %s", dlerror());
#define SYM(field, name)                                                        \
  *(void **)(&g_nccl.field) = dlsym(h, name);                                   \
  if (!g_nccl.field) return fail(CAKE_B200_ENCCL, "libnccl lacks symbol %s", name);
  SYM(GetUniqueId, "ncclGetUniqueId");
  SYM(CommInitRank, "ncclCommInitRank");
  SYM(CommDestroy, "ncclCommDestroy");
  SYM(Send, "ncclSend");
  SYM(Recv, "ncclRecv");
  SYM(GetErrorString, "ncclGetErrorString");
  SYM(GroupStart, "ncclGroupStart");
  SYM(GroupEnd, "ncclGroupEnd");
#undef SYM
  g_nccl.lib = h;
  return CAKE_B200_OK;
}
#define NC(call)                                                                                           \
  do {                                                                                                     \
    ncclResult_t r_ = (call);                                                                              \
    if (r_ != ncclSuccess) return fail(CAKE_B200_ENCCL, "%s:%d %s -> %s", __FILE__, __LINE__, #call, g_nccl.GetErrorString(r_)); \
  } while (0)

// ------------------------------------------------------------------------------------------ handles
struct cake_b200_ctx {
  int device = 0;
  cake_b200_config cfg{};
  int es = 2, sm_count = 148, rot = 0, nqkv = 0;
  cudaStream_t stream = nullptr;
  void *cos_t = nullptr, *sin_t = nullptr;
  // head
  void *embed = nullptr, *ln_f = nullptr, *lm_head = nullptr;
  // decode workspaces
  void *xa = nullptr, *xb = nullptr, *x0 = nullptr, *qkv = nullptr, *y = nullptr, *mm = nullptr, *logits = nullptr;
  float *ws_ml = nullptr, *ws_acc = nullptr, *part_val = nullptr;
  int *part_idx = nullptr, *d_step = nullptr;
  unsigned *attn_counters = nullptr, *argmax_counter = nullptr;
  uint32_t *d_token = nullptr, *token_ring = nullptr, *d_ids = nullptr, *d_pen = nullptr;
  // weight upload pipe: mmapped safetensors -> two pinned staging buffers (filled by a few host
  // threads) -> cudaMemcpy(2D)Async on a copy stream straight into the fused device layouts
  cudaStream_t load_stream = nullptr;
  void *stage[2] = {nullptr, nullptr};
  cudaEvent_t stage_free[2] = {nullptr, nullptr}, load_done = nullptr;
  int stage_cur = 0;
  bool load_pending = false;
  double load_bytes = 0, load_seconds = 0;
  float *samp_p = nullptr, *samp_noise = nullptr;  // sampler scratch: probabilities (vocab) / supplied uniforms
  cake_b200_sampling sampling{};                   // sampler of the decode graph (kind 0 = greedy)
  size_t d_ids_cap = 0, d_pen_cap = 0;
  uint32_t *h_pin = nullptr;  // pinned staging (tokens)
  void *h_pin_x = nullptr;
  size_t h_pin_x_cap = 0;
  int nsplit = 1;
  // prefill workspaces
  size_t pf_rows = 0;
  void *pf_h = nullptr, *pf_qkv = nullptr, *pf_y = nullptr, *pf_x1 = nullptr, *pf_gu = nullptr, *pf_mm = nullptr;
  void *io_x = nullptr;
  size_t io_x_cap = 0;
  // layer-list blocks (fp32 residual stream): operands of the matrix products in D, sized on demand
  size_t sp_rows = 0, sp_in_cols = 0, sp_out_cols = 0, sp_logit_rows = 0;
  void *sp_h = nullptr, *sp_hs = nullptr, *sp_in = nullptr, *sp_a = nullptr, *sp_hn = nullptr;
  float *sp_logits = nullptr;
  int *sp_rows_idx = nullptr;
  // mixer-list blocks: one arena for a step's scratch, grown on demand; vectors kept for cake_b200_stream_inject
  void *mx_ws = nullptr;
  size_t mx_ws_cap = 0;
  void *inject_vec[64] = {};
  const void *inject_src[64] = {};
  // cake_b200_head_load_tables: hashed pair embedding, learned position vectors, the final norm's gain offset
  void *bigram = nullptr, *pos_tab = nullptr;
  int bigram_rows = 0, mul_prev = 0, mul_cur = 0, pos_rows = 0;
  float final_norm_offset = 0.f;
  // the per-layer token inputs of every layer side by side [vocab, side_cols]; the squashing form of the final norm; the ids of
  // the last cake_b200_embed call stay in d_ids (d_ids_n of them) for the layers that read them
  void *side_tab = nullptr, *ln_f_b = nullptr;
  int side_cols = 0, final_norm_kind = 0;
  float final_alpha = 0.f;
  size_t d_ids_n = 0;
  // cake_b200_stream_project: the projection [hidden, 2 hidden] and its operand [rows, 2 hidden] in D
  void *proj_w = nullptr, *proj_ws = nullptr;
  const void *proj_src = nullptr;
  size_t proj_ws_cap = 0;
  // ext blocks with a side mixer: a recurrent side mixer runs on its own stream next to the main mixer (fork after the input
  // projection, join before its output projection); created on first use
  cudaStream_t side_stream = nullptr;
  cudaEvent_t ev_fork = nullptr, ev_join = nullptr;
  // comm
  ncclComm_t comm = nullptr;
  int rank = 0, world = 1;
  // decode graph
  cudaGraphExec_t gexec = nullptr;
  cudaGraph_t graph = nullptr;
  cake_b200_cache *g_cache = nullptr;
  std::vector<int> g_block_idx;
  uint64_t g_kernels = 0;
  int g_rank = 0, g_world = 1;
  long steps_done = 0;
  uint64_t launches = 0;
  bool capturing = false;
  // persistent decode megakernel (decode_mega.cuh); CAKE_B200_PER_OP=1 selects the per-op kernels instead
  bool use_mega = true;
  unsigned long long *gbar = nullptr;   // [0] grid-barrier counter, [1] launch epoch
  MkLayer *mk_tab_dev = nullptr, *mk_tab_host = nullptr, *g_tab_dev = nullptr;
  std::vector<const void *> mk_sig;
  unsigned long long *trace = nullptr;  // CAKE_B200_MEGA_TRACE=1
  unsigned long long *step_trace = nullptr;  // per-step entry / input-acquired / exit stamps of the decode kernels
  unsigned *tickets = nullptr;          // per-phase work-claim counters of the megakernel
  // ring hand-off over NVLink peer memory: inbox = {counter (u64), pad, x[hidden]} in our memory, written by rank-1
  unsigned char *inbox = nullptr, *peer_inbox = nullptr;
  unsigned long long *ring_seq = nullptr;
};
constexpr int TOKEN_RING = 1 << 16;

// Live contexts: a cache may outlive its ctx (handles are freed in any order by foreign hosts), so cache_free only
// touches ctx state when the ctx is still registered here.
static std::mutex g_live_mu;
static std::set<cake_b200_ctx *> g_live_ctx;
static std::atomic<uint64_t> g_cache_gen{1};

struct cake_b200_block {
  cake_b200_ctx *ctx;
  int layer;
  int device = 0;  // copied so that block_free never dereferences a ctx that was destroyed first
  void *wqkv = nullptr, *wo = nullptr, *wgu = nullptr, *wd = nullptr, *ln1 = nullptr, *ln2 = nullptr;
  void *bqkv = nullptr, *qn = nullptr, *kn = nullptr;
  // cake_b200_block_set_variant: the sibling block structures (olmo2 / gemma3 / exaone4 block.rs)
  void *pan = nullptr, *pfn = nullptr;  // post-attention / post-feedforward RmsNorm vectors
  int window = -1;                      // -1: the config's
  bool use_rope = true;
  // cake_b200_block_load_spec: a layer of a layer-list model (fp32 residual stream)
  bool listed = false;
  cake_b200_layer_spec spec{};
  void *w_in = nullptr;    // rows = cat(q, k, gate), zero rows up to n_in_pad
  void *w_out = nullptr;   // [hidden, heads*hd + ff] = o and down side by side along K
  void *g = nullptr, *shift = nullptr, *r1 = nullptr, *r2 = nullptr;
  int n_in = 0, n_in_pad = 0, gate_col = -1, k_out = 0;
  // cake_b200_block_load_mixer: a sequential pre-norm block with a latent-attention / retention / state-space mixer and a
  // routed feed-forward (w_in: the fused input projection, wo: the mixer's output projection, wgu / wd: the shared expert)
  bool mixer = false;
  cake_b200_mixer_spec ms{};
  void *m_dkv_norm = nullptr, *m_uk = nullptr, *m_uv = nullptr, *m_ukt = nullptr;  // m_ukt: uk per head as [kv_rank, dim]
  void *m_conv = nullptr, *m_conv_b = nullptr, *m_dt_bias = nullptr, *m_a_log = nullptr, *m_d = nullptr, *m_norm = nullptr;
  void *m_router = nullptr, *m_corr = nullptr, *m_eg = nullptr, *m_ed = nullptr;
  float *m_cos = nullptr, *m_sin = nullptr, *m_decay = nullptr;
  int m_rope_rows = 0;
  // the block structure switches of cake_b200_mixer_spec (norm_offset, post norms, canon_taps, side, dense_ff) and the delta /
  // talking-attention / matrix-memory mixers: `ext` blocks run enqueue_ext_layer.  A side mixer's own tensors live in a nested
  // block; its projections are rows of this block's w_in.  pc[]: the column of each projection part in the step's `proj`.
  bool ext = false;
  cake_b200_block *side = nullptr;
  void *post1 = nullptr, *post2 = nullptr, *canon = nullptr, *b_in = nullptr;
  void *m_ob = nullptr, *m_talk = nullptr, *m_branch = nullptr, *m_ib = nullptr, *m_fb = nullptr;
  float *m_bias = nullptr;   // [m_bias_len, heads] fp32: the distance bias by distance
  int m_bias_len = 0;
  int pc[6] = {0, 0, 0, 0, 0, 0};
  // sink attention / windowed latent attention; the offsets of the squashing norms; the per-layer token input
  void *m_sink = nullptr, *m_dq_norm = nullptr, *m_uq = nullptr;
  void *ln1_b = nullptr, *post1_b = nullptr, *ln2_b = nullptr, *post2_b = nullptr;
  void *sd_gate = nullptr, *sd_proj = nullptr, *sd_norm = nullptr;
  bool variant() const { return !ln1 || !ln2 || pan || pfn || window >= 0 || !use_rope || ctx->cfg.pre_reshape_qk_norm; }
};

struct cake_b200_cache {
  cake_b200_ctx *ctx;
  int batch, cap;
  int device = 0;
  uint64_t gen = 0;  // unique per cache object: part of the megakernel layer-table signature (addresses can be reused)
  std::vector<void *> k, v;
  std::vector<int> len;
  int *d_pos = nullptr;
  // layer-list blocks: the row width the layer's K cache was allocated with, and the token-shift state (the last h of the
  // previous call, fp32 [batch, hidden]) in two buffers that swap roles every call
  std::vector<int> kv_heads, kv_hd;
  std::vector<float *> shift_state[2];
  std::vector<int> shift_cur;
  // mixer-list blocks: recurrent state [batch, heads, dk, dv] fp32 and the convolution's last taps - 1 inputs, per block_idx
  std::vector<float *> rec_state;
  std::vector<void *> conv_hist;
  // ext blocks: k / v / rec_state / conv_hist / rec_aux have a second entry per block_idx (index n_layers + block_idx) for a
  // side mixer; rec_aux: the normaliser and running maximum of a matrix memory [batch, heads, dk + 1] fp32; canon_hist: the
  // last canon_taps - 1 normed inputs of the block [batch, taps - 1, hidden] fp32
  std::vector<float *> rec_aux, canon_hist;
  std::vector<void *> vt;   // talking attention on the tensor cores: the values once more, [batch, kv_heads, vdim, cap_t] with positions innermost
  // cake_b200_embed_at: the last token of every batch row and the position the embedding has reached
  std::vector<uint32_t> last_tok;
  int embed_len = 0;
};

template <typename U> struct TypeTag { typedef U type; };
template <typename F> static inline int dispatch_T(int dtype, F &&f) {
  if (dtype != CAKE_B200_F16) return f(TypeTag<__nv_bfloat16>{});  // an fp32 layer-list model hands its samplers bf16 logits
  return f(TypeTag<__half>{});
}
template <typename F> static inline int dispatch_T3(int dtype, F &&f) {
  if (dtype == CAKE_B200_F32) return f(TypeTag<float>{});
  return dispatch_T(dtype, f);
}
#define DISPATCH_T3(dtype, ...) dispatch_T3((dtype), __VA_ARGS__)
// usage: DISPATCH_T(dtype, [&](auto tag_) -> int { typedef typename decltype(tag_)::type T; ... })
#define DISPATCH_T(dtype, ...) dispatch_T((dtype), __VA_ARGS__)
#define T_LAMBDA [&](auto tag_) -> int

// (head_dim, query heads per kv head) combinations the megakernel is instantiated for
#define MK_FOR_ALL(X) X(16, 2) X(16, 4) X(64, 2) X(64, 4) X(128, 1) X(128, 2) X(128, 4) X(128, 8)

// ------------------------------------------------------------------------------------------ launch helper (PDL)
template <typename... KArgs, typename... Args>
static int launch_pdl(cake_b200_ctx *c, void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, Args... args) {
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = c->stream;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = at;
  cfg.numAttrs = 1;
  CU(cudaLaunchKernelEx(&cfg, kern, KArgs(args)...));
  if (c->capturing) c->g_kernels++;
  else c->launches++;
  return CAKE_B200_OK;
}

// the same with a thread-block cluster of `cluster` CTAs along x (TMA multicast between the CTAs of a pair)
template <typename... KArgs, typename... Args>
static int launch_cluster_pdl(cake_b200_ctx *c, void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, unsigned cluster, Args... args) {
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = c->stream;
  cudaLaunchAttribute at[2];
  at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[0].val.programmaticStreamSerializationAllowed = 1;
  at[1].id = cudaLaunchAttributeClusterDimension;
  at[1].val.clusterDim.x = cluster;
  at[1].val.clusterDim.y = 1;
  at[1].val.clusterDim.z = 1;
  cfg.attrs = at;
  cfg.numAttrs = 2;
  CU(cudaLaunchKernelEx(&cfg, kern, KArgs(args)...));
  if (c->capturing) c->g_kernels++;
  else c->launches++;
  return CAKE_B200_OK;
}

// ------------------------------------------------------------------------------------------ GEMV plan + launch
struct GemvPlan {
  int KC, RS, WPR, RPW, n_stages, max_rows, grid;
  size_t smem;
};
static int plan_gemv(const cake_b200_ctx *c, int N, int K, int G, GemvPlan *p) {
  const int es = c->es;
  if (K % 64 != 0 || N % G != 0) return fail(CAKE_B200_EINVAL, "gemv: K=%d must be a multiple of 64, N=%d of %d", K, N, G);
  // segment: whole rows up to 16 KB, else the row is halved until it is (K=14336 -> 2 x 14 KB)
  int KC = K;
  while ((size_t)KC * es > 16384 && (KC / 2) % 64 == 0) KC /= 2;
  const size_t seg = (size_t)KC * es;
  // column slices: keep >= 64 16-byte vectors per warp per row where the row is long enough
  int WPR = 1;
  while (WPR < 8 && (KC / 8) / (WPR * 2) >= 64) WPR *= 2;
  if (WPR > 4) WPR = 4;
  const int slots = GEMV_CONSUMER_WARPS / WPR;
  int RPW = 1;  // rows per warp per stage: grow the stage towards 32 KB
  while (RPW < 4 && (size_t)(slots * RPW * 2) * seg <= 32768) RPW *= 2;
  const int RS = slots * RPW;
  const int units = N / G;
  const int grid = units < c->sm_count ? units : c->sm_count;
  const int max_rows = (units / grid + 1) * G;
  // two CTAs (this kernel + its PDL successor) must fit in one SM's 227 KB
  const size_t budget = ((size_t)K * es > 16384 ? 116 : 108) * 1024;
  int ns = GEMV_MAX_STAGES;
  while (ns > 2 && gemv_smem_bytes(K, KC, RS, WPR, ns, max_rows, es) > budget) ns--;
  const size_t smem = gemv_smem_bytes(K, KC, RS, WPR, ns, max_rows, es);
  if (smem > 227 * 1024) return fail(CAKE_B200_EINVAL, "gemv: N=%d K=%d needs %zu B of shared memory", N, K, smem);
  *p = GemvPlan{KC, RS, WPR, RPW, ns, max_rows, grid, smem};
  return CAKE_B200_OK;
}

template <typename T, int EPI> static int launch_gemv_T(cake_b200_ctx *c, GemvArgs a, const GemvPlan &p) {
  a.KC = p.KC;
  a.RS = p.RS;
  a.WPR = p.WPR;
  a.n_stages = p.n_stages;
  a.max_rows = p.max_rows;
  dim3 grid(p.grid), block(GEMV_THREADS);
  switch (p.RPW) {
    case 1: return launch_pdl(c, gemv_kernel<T, EPI, 1>, grid, block, p.smem, a);
    case 2: return launch_pdl(c, gemv_kernel<T, EPI, 2>, grid, block, p.smem, a);
    default: return launch_pdl(c, gemv_kernel<T, EPI, 4>, grid, block, p.smem, a);
  }
}
template <int EPI> static int launch_gemv(cake_b200_ctx *c, GemvArgs a) {
  GemvPlan p;
  RC(plan_gemv(c, a.N, a.K, EPI == EPI_SWIGLU ? 2 : 1, &p));
  return DISPATCH_T(c->cfg.dtype, T_LAMBDA {
      typedef typename decltype(tag_)::type T; return launch_gemv_T<T, EPI>(c, a, p); });
}

template <typename T> static int set_smem_attrs_T() {
  const int maxs = 227 * 1024;
  // max-shared carveout so that a kernel and its programmatic-dependent successor co-reside on an SM
#define SETA1(EPI, R)                                                                                          \
  CU(cudaFuncSetAttribute(gemv_kernel<T, EPI, R>, cudaFuncAttributeMaxDynamicSharedMemorySize, maxs));         \
  CU(cudaFuncSetAttribute(gemv_kernel<T, EPI, R>, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared));
#define SETA(EPI) SETA1(EPI, 1) SETA1(EPI, 2) SETA1(EPI, 4)
  SETA(EPI_PLAIN) SETA(EPI_RESIDUAL) SETA(EPI_SWIGLU) SETA(EPI_ARGMAX)
#undef SETA
#undef SETA1
#define SETB(HD)                                                                                                  \
  CU(cudaFuncSetAttribute(attn_decode_kernel<T, HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, maxs - 4096)); /* static smem counts too */         \
  CU(cudaFuncSetAttribute(attn_decode_kernel<T, HD>, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared));
  SETB(16) SETB(32) SETB(64) SETB(128) SETB(256)
#undef SETB
#define SETC(HD, G)                                                                                                  \
  CU(cudaFuncSetAttribute(decode_mega_kernel<T, HD, G>, cudaFuncAttributeMaxDynamicSharedMemorySize, maxs - 4096));  \
  CU(cudaFuncSetAttribute(decode_mega_kernel<T, HD, G>, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared));
  MK_FOR_ALL(SETC)
#undef SETC
  CU(cudaFuncSetAttribute(attn_prefill_mma_kernel<T, 128>, cudaFuncAttributeMaxDynamicSharedMemorySize, 4 * FA_BN * 128 * 2));
  CU(cudaFuncSetAttribute(attn_prefill_mma_kernel<T, 64>, cudaFuncAttributeMaxDynamicSharedMemorySize, 4 * FA_BN * 64 * 2));
  CU(cudaFuncSetAttribute(attn_prefill_tc_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, FT_SMEM_BYTES));
  CU(cudaFuncSetAttribute(attn_prefill_tc_kernel<T>, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared));
#define SETT(EPI)                                                                                                                  \
  CU(cudaFuncSetAttribute(gemm_tc_kernel<T, EPI, 128>, cudaFuncAttributeMaxDynamicSharedMemorySize, TcCfg<128>::SMEM_BYTES));      \
  CU(cudaFuncSetAttribute(gemm_tc_kernel<T, EPI, 256>, cudaFuncAttributeMaxDynamicSharedMemorySize, TcCfg<256>::SMEM_BYTES));      \
  CU(cudaFuncSetAttribute(gemm_tc_kernel<T, EPI, 256, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, TcCfg<256>::SMEM_BYTES));
  SETT(TCE_PLAIN) SETT(TCE_RESIDUAL) SETT(TCE_SWIGLU) SETT(TCE_RESIDUAL_F32) SETT(TCE_SOFTCAP_F32)
  CU(cudaFuncSetAttribute(attn_window_tc_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, FT_SMEM_BYTES));
  CU(cudaFuncSetAttribute(attn_window_tc_kernel<T>, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared));
#define SETW(HD) CU(cudaFuncSetAttribute(attn_window_mma_kernel<T, HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, wm_smem_bytes<HD>()));
  SETW(32) SETW(64) SETW(96) SETW(128)
#undef SETW
#undef SETT
  return CAKE_B200_OK;
}

// ------------------------------------------------------------------------------------------ context
static void rope_tables_host(const cake_b200_config &c, std::vector<float> &cs, std::vector<float> &sn, int rot) {
  // cache.rs:43-96 (same arithmetic the reference performs on the host; computed once per ctx)
  const int half = rot / 2;
  std::vector<float> theta(half > 0 ? half : 1);
  for (int j = 0; j < half; j++) theta[j] = 1.0f / powf(c.rope_theta, (float)(2 * j) / (float)rot);
  if (c.rope_llama3 && c.rope_orig_max > 0) {
    const float old = (float)c.rope_orig_max;
    const float low_wl = old / c.rope_low, high_wl = old / c.rope_high;
    for (int j = 0; j < half; j++) {
      const float wl = 2.0f * 3.14159265358979323846f / theta[j];
      if (wl < high_wl) {
      } else if (wl > low_wl) {
        theta[j] /= c.rope_factor;
      } else {
        const float smooth = (old / wl - c.rope_low) / (c.rope_high - c.rope_low);
        theta[j] = (1.0f - smooth) * (theta[j] / c.rope_factor) + smooth * theta[j];
      }
    }
  }
  cs.resize((size_t)c.max_seq * half);
  sn.resize((size_t)c.max_seq * half);
  for (int p = 0; p < c.max_seq; p++)
    for (int j = 0; j < half; j++) {
      const float ang = (float)p * theta[j];
      cs[(size_t)p * half + j] = cosf(ang);
      sn[(size_t)p * half + j] = sinf(ang);
    }
}
static void f32_to_D(const std::vector<float> &src, std::vector<uint16_t> &dst, int dtype) {
  dst.resize(src.size());
  for (size_t i = 0; i < src.size(); i++) {
    if (dtype == CAKE_B200_BF16) {
      bf16 v = __float2bfloat16_rn(src[i]);
      memcpy(&dst[i], &v, 2);
    } else {
      __half v = __float2half_rn(src[i]);
      memcpy(&dst[i], &v, 2);
    }
  }
}

extern "C" int cake_b200_ctx_create(int device, const cake_b200_config *cfg, cake_b200_ctx **out) {
  if (!cfg || !out) return fail(CAKE_B200_EINVAL, "null argument");
  cake_b200_config listed_cfg;
  if (cfg->layer_list) {
    // every per-layer size comes with the layers; the fields the Llama-family paths size their workspaces by are set to the
    // smallest legal values so that those workspaces exist (samplers, token staging) but cost nothing
    if (cfg->dtype != CAKE_B200_BF16 && cfg->dtype != CAKE_B200_F16 && cfg->dtype != CAKE_B200_F32)
      return fail(CAKE_B200_EINVAL, "dtype %d unsupported (bf16=0, f16=1, f32=2)", cfg->dtype);
    if (cfg->hidden < 1 || cfg->n_layers < 1 || cfg->vocab < 1 || cfg->max_seq < 1) return fail(CAKE_B200_EINVAL, "config dimensions must be positive");
    listed_cfg = *cfg;
    listed_cfg.inter = 64; listed_cfg.n_heads = 1; listed_cfg.n_kv_heads = 1; listed_cfg.head_dim = 16;
    listed_cfg.partial_rotary = 0.f; listed_cfg.rope_llama3 = 0; listed_cfg.sliding_window = 0;
    cfg = &listed_cfg;
  } else {
  if (cfg->dtype != CAKE_B200_BF16 && cfg->dtype != CAKE_B200_F16)
    return fail(CAKE_B200_EINVAL, "dtype %d unsupported (bf16=0, f16=1; f32 is for layer-list models)", cfg->dtype);
  if (cfg->hidden < 1 || cfg->inter < 1 || cfg->n_heads < 1 || cfg->n_kv_heads < 1 || cfg->n_layers < 1 || cfg->vocab < 1 || cfg->max_seq < 1)
    return fail(CAKE_B200_EINVAL, "config dimensions must be positive");
  if (cfg->n_heads % cfg->n_kv_heads != 0 || cfg->n_heads / cfg->n_kv_heads > ATTN_MAX_G)
    return fail(CAKE_B200_EINVAL, "n_heads/n_kv_heads must be an integer <= %d", ATTN_MAX_G);
  if (cfg->head_dim != 16 && cfg->head_dim != 32 && cfg->head_dim != 64 && cfg->head_dim != 128 && cfg->head_dim != 256)
    return fail(CAKE_B200_EINVAL, "head_dim %d unsupported (16/32/64/128/256)", cfg->head_dim);
  if (cfg->hidden % 64 || cfg->inter % 64 || (cfg->n_heads * cfg->head_dim) % 64)
    return fail(CAKE_B200_EINVAL, "hidden, intermediate and n_heads*head_dim must be multiples of 64");
  }
  int ndev = 0;
  CU(cudaGetDeviceCount(&ndev));
  if (ndev == 0) return fail(CAKE_B200_ECUDA, "no CUDA device: libcake_b200 has no CPU fallback");
  CU(cudaSetDevice(device));
  cudaDeviceProp prop;
  CU(cudaGetDeviceProperties(&prop, device));
  if (prop.major != 10) return fail(CAKE_B200_ECUDA, "device %d is sm_%d%d; this library is built for sm_100a only", device, prop.major, prop.minor);
  auto *c = new cake_b200_ctx();
  // any failure below returns through CU / RC: release what was set up so far (ctx_destroy tolerates a half-built ctx)
  struct Guard { cake_b200_ctx *c; ~Guard() { if (c) { cake_b200_ctx_destroy(c); (void)cudaGetLastError(); } } } guard{c};
  c->device = device;
  c->cfg = *cfg;
  c->es = cfg->dtype == CAKE_B200_F32 ? 4 : 2;
  c->sm_count = prop.multiProcessorCount;
  c->rot = (int)((float)cfg->head_dim * cfg->partial_rotary);
  c->nqkv = (cfg->n_heads + 2 * cfg->n_kv_heads) * cfg->head_dim;
  CU(cudaStreamCreateWithFlags(&c->stream, cudaStreamNonBlocking));
  RC(set_smem_attrs_T<__nv_bfloat16>());
  RC(set_smem_attrs_T<__half>());
  // RoPE tables -> D
  std::vector<float> cs, sn;
  rope_tables_host(*cfg, cs, sn, c->rot);
  std::vector<uint16_t> cd, sd;
  f32_to_D(cs, cd, cfg->dtype == CAKE_B200_F16 ? CAKE_B200_F16 : CAKE_B200_BF16);
  f32_to_D(sn, sd, cfg->dtype == CAKE_B200_F16 ? CAKE_B200_F16 : CAKE_B200_BF16);
  const size_t tb = cd.size() * 2 + 16;
  CU(cudaMalloc(&c->cos_t, tb));
  CU(cudaMalloc(&c->sin_t, tb));
  CU(cudaMemcpy(c->cos_t, cd.data(), cd.size() * 2, cudaMemcpyHostToDevice));
  CU(cudaMemcpy(c->sin_t, sd.data(), sd.size() * 2, cudaMemcpyHostToDevice));
  // decode workspaces
  const int H = cfg->hidden, I = cfg->inter, nh = cfg->n_heads, hd = cfg->head_dim;
  c->nsplit = c->sm_count / cfg->n_kv_heads;
  if (c->nsplit < 1) c->nsplit = 1;
  if (c->nsplit > ATTN_MAX_SPLIT) c->nsplit = ATTN_MAX_SPLIT;
  CU(cudaMalloc(&c->xa, (size_t)H * 2));
  CU(cudaMalloc(&c->xb, (size_t)H * 2));
  CU(cudaMalloc(&c->x0, (size_t)H * 2));
  CU(cudaMalloc(&c->qkv, (size_t)c->nqkv * 2));
  CU(cudaMalloc(&c->y, (size_t)nh * hd * 2));
  CU(cudaMalloc(&c->mm, (size_t)I * 2));
  CU(cudaMalloc(&c->logits, (size_t)cfg->vocab * 2));
  CU(cudaMalloc(&c->ws_ml, (size_t)nh * c->nsplit * 2 * 4));
  CU(cudaMalloc(&c->ws_acc, (size_t)nh * c->nsplit * hd * 4));
  CU(cudaMalloc(&c->attn_counters, (size_t)cfg->n_kv_heads * 4));
  CU(cudaMemset(c->attn_counters, 0, (size_t)cfg->n_kv_heads * 4));
  CU(cudaMalloc(&c->part_val, 1024 * 4));
  CU(cudaMalloc(&c->part_idx, 1024 * 4));
  CU(cudaMalloc(&c->argmax_counter, 4));
  CU(cudaMemset(c->argmax_counter, 0, 4));
  CU(cudaMalloc(&c->d_token, 4));
  CU(cudaMalloc(&c->d_step, 4));
  CU(cudaMemset(c->d_step, 0, 4));
  CU(cudaMalloc(&c->token_ring, (size_t)TOKEN_RING * 4));
  CU(cudaMallocHost(&c->h_pin, 64 * 4));
  CU(cudaMalloc(&c->gbar, 16));
  CU(cudaMemset(c->gbar, 0, 16));
  CU(cudaMalloc(&c->tickets, sizeof(unsigned) * (4 * MK_MAX_LAYERS + 4)));
  CU(cudaMalloc(&c->ring_seq, 8));
  CU(cudaMemset(c->ring_seq, 0, 8));
  CU(cudaMalloc(&c->step_trace, sizeof(unsigned long long) * MK_STEP_RING * 8));
  CU(cudaMemset(c->step_trace, 0, sizeof(unsigned long long) * MK_STEP_RING * 8));
  CU(cudaMalloc(&c->mk_tab_dev, sizeof(MkLayer) * MK_MAX_LAYERS));
  CU(cudaMalloc(&c->g_tab_dev, sizeof(MkLayer) * MK_MAX_LAYERS));
  CU(cudaMallocHost(&c->mk_tab_host, sizeof(MkLayer) * MK_MAX_LAYERS));
  {
    const char *e = getenv("CAKE_B200_PER_OP");
    c->use_mega = !(e && e[0] == '1');
    const char *t = getenv("CAKE_B200_MEGA_TRACE");
    if (t && t[0] == '1') {
      CU(cudaMalloc(&c->trace, 8 * 4096));
      CU(cudaMemset(c->trace, 0, 8 * 4096));
    }
  }
  {
    std::lock_guard<std::mutex> lk(g_live_mu);
    g_live_ctx.insert(c);
  }
  guard.c = nullptr;
  *out = c;
  return CAKE_B200_OK;
}

extern "C" void cake_b200_ctx_destroy(cake_b200_ctx *c) {
  if (!c) return;
  {
    std::lock_guard<std::mutex> lk(g_live_mu);
    g_live_ctx.erase(c);
  }
  cudaSetDevice(c->device);
  cudaStreamSynchronize(c->stream);
  if (c->gexec) cudaGraphExecDestroy(c->gexec);
  if (c->graph) cudaGraphDestroy(c->graph);
  if (c->comm && g_nccl.CommDestroy) g_nccl.CommDestroy(c->comm);
  if (c->peer_inbox) cudaIpcCloseMemHandle(c->peer_inbox);
  void *bufs[] = {c->cos_t, c->sin_t, c->embed, c->ln_f, c->xa, c->xb, c->qkv, c->y, c->mm, c->logits, c->ws_ml,
                  c->ws_acc, c->part_val, c->part_idx, c->d_step, c->attn_counters, c->argmax_counter, c->d_token,
                  c->token_ring, c->d_ids, c->d_pen, c->pf_h, c->pf_qkv, c->pf_y, c->pf_x1, c->pf_gu, c->pf_mm, c->io_x,
                  c->gbar, c->mk_tab_dev, c->g_tab_dev, c->tickets, c->ring_seq, c->inbox, c->step_trace, c->trace,
                  c->samp_p, c->samp_noise, c->x0, c->sp_h, c->sp_hs, c->sp_in, c->sp_a, c->sp_hn, c->sp_logits, c->sp_rows_idx, c->mx_ws};
  for (void *b : bufs)
    if (b) cudaFree(b);
  if (c->bigram) cudaFree(c->bigram);
  if (c->pos_tab) cudaFree(c->pos_tab);
  for (void *b : {c->side_tab, c->ln_f_b, c->proj_w, c->proj_ws})
    if (b) cudaFree(b);
  for (void *b : c->inject_vec)
    if (b) cudaFree(b);
  if (c->lm_head && c->lm_head != c->embed) cudaFree(c->lm_head);
  for (int i = 0; i < 2; i++) {
    if (c->stage[i]) cudaFreeHost(c->stage[i]);
    if (c->stage_free[i]) cudaEventDestroy(c->stage_free[i]);
  }
  if (c->load_done) cudaEventDestroy(c->load_done);
  if (c->ev_fork) cudaEventDestroy(c->ev_fork);
  if (c->ev_join) cudaEventDestroy(c->ev_join);
  if (c->side_stream) { cudaStreamSynchronize(c->side_stream); cudaStreamDestroy(c->side_stream); }
  if (c->load_stream) { cudaStreamSynchronize(c->load_stream); cudaStreamDestroy(c->load_stream); }
  if (c->h_pin) cudaFreeHost(c->h_pin);
  if (c->h_pin_x) cudaFreeHost(c->h_pin_x);
  if (c->mk_tab_host) cudaFreeHost(c->mk_tab_host);
  cudaStreamDestroy(c->stream);
  delete c;
}
extern "C" int cake_b200_sync(cake_b200_ctx *c) {
  if (!c) return fail(CAKE_B200_EINVAL, "null argument");
  CU(cudaSetDevice(c->device));
  RC(wait_loads(c));
  if (c->load_stream) CU(cudaStreamSynchronize(c->load_stream));
  CU(cudaStreamSynchronize(c->stream));
  return CAKE_B200_OK;
}
extern "C" void *cake_b200_stream(cake_b200_ctx *c) { return c ? (void *)c->stream : nullptr; }
extern "C" int cake_b200_launch_count(cake_b200_ctx *c, uint64_t *k) {
  if (!c || !k) return fail(CAKE_B200_EINVAL, "null argument");
  *k = c->launches;
  return CAKE_B200_OK;
}

extern "C" int cake_b200_dev_alloc(cake_b200_ctx *c, size_t bytes, void **out) {
  if (!c || !out) return fail(CAKE_B200_EINVAL, "null argument");
  CU(cudaSetDevice(c->device));
  CU(cudaMalloc(out, bytes ? bytes : 16));
  return CAKE_B200_OK;
}
extern "C" int cake_b200_dev_free(cake_b200_ctx *c, void *p) {
  if (!c) return fail(CAKE_B200_EINVAL, "null argument");
  CU(cudaSetDevice(c->device));
  CU(cudaStreamSynchronize(c->stream));
  CU(cudaFree(p));
  return CAKE_B200_OK;
}

// ------------------------------------------------------------------------------------------ weight upload pipe
constexpr size_t STAGE_BYTES = (size_t)64 << 20;
constexpr int STAGE_THREADS = 6;
static int pipe_init(cake_b200_ctx *c) {
  if (c->load_stream) return CAKE_B200_OK;
  CU(cudaStreamCreateWithFlags(&c->load_stream, cudaStreamNonBlocking));
  for (int i = 0; i < 2; i++) {
    CU(cudaMallocHost(&c->stage[i], STAGE_BYTES));
    CU(cudaEventCreateWithFlags(&c->stage_free[i], cudaEventDisableTiming));
  }
  CU(cudaEventCreateWithFlags(&c->load_done, cudaEventDisableTiming));
  return CAKE_B200_OK;
}
// host rows [r0, r1) of width bytes (source pitch spitch) -> packed staging buffer, split over a few threads: one thread
// tops out at ~6 GB/s out of the page cache, far below what the PCIe link takes
static void stage_rows(char *dst, const char *src, size_t spitch, size_t width, size_t rows) {
  const size_t total = rows * width;
  int nt = total >= ((size_t)4 << 20) ? STAGE_THREADS : 1;
  if (nt == 1) {
    for (size_t r = 0; r < rows; r++) memcpy(dst + r * width, src + r * spitch, width);
    return;
  }
  std::vector<std::thread> th;
  if (spitch == width) {  // contiguous: split by bytes
    for (int t = 0; t < nt; t++) {
      const size_t a = total * t / nt, b = total * (t + 1) / nt;
      th.emplace_back([=]() { memcpy(dst + a, src + a, b - a); });
    }
  } else {
    for (int t = 0; t < nt; t++) {
      const size_t a = rows * t / nt, b = rows * (t + 1) / nt;
      th.emplace_back([=]() { for (size_t r = a; r < b; r++) memcpy(dst + r * width, src + r * spitch, width); });
    }
  }
  for (auto &x : th) x.join();
}
// dst[r * dpitch .. + width) = src[r * spitch .. + width) for r < rows (rows == 1: a plain copy).  Device sources
// (synthetic checkpoints generated on the GPU) are copied device-to-device on the same stream.
static int pipe_copy(cake_b200_ctx *c, void *dst, size_t dpitch, const void *src, size_t spitch, size_t width, size_t rows) {
  RC(pipe_init(c));
  cudaPointerAttributes at{};
  const bool dev_src = (cudaPointerGetAttributes(&at, src) == cudaSuccess) && (at.type == cudaMemoryTypeDevice || at.type == cudaMemoryTypeManaged);
  (void)cudaGetLastError();
  if (dev_src) {
    // written by someone else's stream (torch): copy on the legacy default stream, which orders after that work, and
    // wait — the caller may free the source as soon as we return
    CU(cudaMemcpy2D(dst, dpitch, src, spitch, width, rows, cudaMemcpyDeviceToDevice));
    CU(cudaStreamSynchronize(0));
    return CAKE_B200_OK;
  }
  const auto t0 = std::chrono::steady_clock::now();
  if (rows == 1 && width > STAGE_BYTES) {  // a long contiguous tensor: treat it as rows of 1 MB
    const size_t rw = (size_t)1 << 20, full = width / rw;
    if (full) RC(pipe_copy(c, dst, rw, src, rw, rw, full));
    if (width % rw) RC(pipe_copy(c, (char *)dst + full * rw, width % rw, (const char *)src + full * rw, width % rw, width % rw, 1));
    return CAKE_B200_OK;
  }
  const size_t rows_per = std::max<size_t>(1, STAGE_BYTES / width);
  for (size_t r0 = 0; r0 < rows; r0 += rows_per) {
    const size_t nr = std::min(rows_per, rows - r0);
    const int b = c->stage_cur;
    CU(cudaEventSynchronize(c->stage_free[b]));  // the DMA that last read this buffer has finished
    stage_rows((char *)c->stage[b], (const char *)src + r0 * spitch, spitch, width, nr);
    CU(cudaMemcpy2DAsync((char *)dst + r0 * dpitch, dpitch, c->stage[b], width, width, nr, cudaMemcpyHostToDevice, c->load_stream));
    CU(cudaEventRecord(c->stage_free[b], c->load_stream));
    c->stage_cur ^= 1;
  }
  c->load_bytes += (double)width * rows;
  c->load_seconds += std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
  return CAKE_B200_OK;
}
static int pipe_mark(cake_b200_ctx *c) {  // compute must not start before the uploads issued so far have landed
  CU(cudaEventRecord(c->load_done, c->load_stream));
  c->load_pending = true;
  return CAKE_B200_OK;
}
static int wait_loads(cake_b200_ctx *c) {
  if (c->load_pending) {
    CU(cudaStreamWaitEvent(c->stream, c->load_done, 0));
    c->load_pending = false;
  }
  return CAKE_B200_OK;
}

// ------------------------------------------------------------------------------------------ blocks
static int upload(cake_b200_ctx *c, void **dst, const void *src, size_t bytes) {
  CU(cudaMalloc(dst, bytes + 16));
  return pipe_copy(c, *dst, bytes, src, bytes, bytes, 1);
}

extern "C" void cake_b200_block_free(cake_b200_block *b);
extern "C" int cake_b200_block_load(cake_b200_ctx *c, int layer_idx, const void *q, const void *k, const void *v,
                                    const void *o, const void *gate, const void *up, const void *down, const void *ln1,
                                    const void *ln2, const void *q_bias, const void *k_bias, const void *v_bias,
                                    const void *q_norm, const void *k_norm, cake_b200_block **out) {
  if (!c || !q || !k || !v || !o || !gate || !up || !down || !out) return fail(CAKE_B200_EINVAL, "null weight pointer");  // ln1 / ln2 may be NULL (OLMo2: no pre-norms)
  if (c->cfg.qkv_bias && (!q_bias || !k_bias || !v_bias)) return fail(CAKE_B200_EINVAL, "config has qkv_bias but a bias pointer is null");
  if (c->cfg.qk_norm && (!q_norm || !k_norm)) return fail(CAKE_B200_EINVAL, "config has qk_norm but a norm pointer is null");
  CU(cudaSetDevice(c->device));
  const size_t es = c->es, H = c->cfg.hidden, I = c->cfg.inter, hd = c->cfg.head_dim;
  const size_t sq = (size_t)c->cfg.n_heads * hd, skv = (size_t)c->cfg.n_kv_heads * hd;
  auto *b = new cake_b200_block{c, layer_idx, c->device};
  const int rc = [&]() -> int {  // on any failure (e.g. out of memory half way through a shard) nothing is leaked
  // attention.rs:109-113: Wqkv = cat([q,k,v], 0)
  CU(cudaMalloc(&b->wqkv, (sq + 2 * skv) * H * es + 16));
  RC(pipe_copy(c, b->wqkv, sq * H * es, q, sq * H * es, sq * H * es, 1));
  RC(pipe_copy(c, (char *)b->wqkv + sq * H * es, skv * H * es, k, skv * H * es, skv * H * es, 1));
  RC(pipe_copy(c, (char *)b->wqkv + (sq + skv) * H * es, skv * H * es, v, skv * H * es, skv * H * es, 1));
  RC(upload(c, &b->wo, o, H * sq * es));
  // mlp.rs:43-45 fuses gate|up by cat; here the fused matrix is ROW-INTERLEAVED (row 2i = gate_i,
  // row 2i+1 = up_i) so that silu(gate_i)*up_i is local to one warp's epilogue.  Numerically identical.
  CU(cudaMalloc(&b->wgu, 2 * I * H * es + 16));
  RC(pipe_copy(c, b->wgu, 2 * H * es, gate, H * es, H * es, I));               // the row interleave is done by the DMA engine
  RC(pipe_copy(c, (char *)b->wgu + H * es, 2 * H * es, up, H * es, H * es, I));
  RC(upload(c, &b->wd, down, H * I * es));
  if (ln1) RC(upload(c, &b->ln1, ln1, H * es));
  if (ln2) RC(upload(c, &b->ln2, ln2, H * es));
  if (c->cfg.qkv_bias) {
    CU(cudaMalloc(&b->bqkv, (sq + 2 * skv) * es + 16));
    RC(pipe_copy(c, b->bqkv, sq * es, q_bias, sq * es, sq * es, 1));
    RC(pipe_copy(c, (char *)b->bqkv + sq * es, skv * es, k_bias, skv * es, skv * es, 1));
    RC(pipe_copy(c, (char *)b->bqkv + (sq + skv) * es, skv * es, v_bias, skv * es, skv * es, 1));
  }
  if (c->cfg.qk_norm) {
    RC(upload(c, &b->qn, q_norm, (c->cfg.pre_reshape_qk_norm ? sq : hd) * es));   // attention.rs:121-122
    RC(upload(c, &b->kn, k_norm, (c->cfg.pre_reshape_qk_norm ? skv : hd) * es));
  }
  return pipe_mark(c);
  }();
  if (rc != CAKE_B200_OK) {
    cake_b200_block_free(b);
    return rc;
  }
  *out = b;
  return CAKE_B200_OK;
}
extern "C" void cake_b200_block_free(cake_b200_block *b) {
  if (!b) return;
  cudaSetDevice(b->device);
  void *bufs[] = {b->wqkv, b->wo, b->wgu, b->wd, b->ln1, b->ln2, b->bqkv, b->qn, b->kn, b->pan, b->pfn,
                  b->w_in, b->w_out, b->g, b->shift, b->r1, b->r2, b->m_dkv_norm, b->m_uk, b->m_uv, b->m_ukt, b->m_conv, b->m_conv_b, b->m_dt_bias,
                  b->m_a_log, b->m_d, b->m_norm, b->m_router, b->m_corr, b->m_eg, b->m_ed, b->m_cos, b->m_sin, b->m_decay,
                  b->post1, b->post2, b->canon, b->b_in, b->m_ob, b->m_talk, b->m_branch, b->m_ib, b->m_fb, b->m_bias,
                  b->m_sink, b->m_dq_norm, b->m_uq, b->ln1_b, b->post1_b, b->ln2_b, b->post2_b, b->sd_gate, b->sd_proj, b->sd_norm};
  for (void *p : bufs)
    if (p) cudaFree(p);  // cudaFree synchronises with outstanding work
  if (b->side) cake_b200_block_free(b->side);
  (void)cudaGetLastError();
  delete b;
}
extern "C" int cake_b200_block_layer(const cake_b200_block *b) { return b ? b->layer : -1; }
extern "C" int cake_b200_block_set_variant(cake_b200_block *b, const cake_b200_block_variant *v) {
  if (!b || !v) return fail(CAKE_B200_EINVAL, "null argument");
  if (v->sliding_window < -1) return fail(CAKE_B200_EINVAL, "sliding_window %d (use -1 for the config's, 0 for none)", v->sliding_window);
  cake_b200_ctx *c = b->ctx;
  CU(cudaSetDevice(c->device));
  const size_t bytes = (size_t)c->cfg.hidden * c->es;
  if (v->post_attention_norm) {
    if (b->pan) { cudaFree(b->pan); b->pan = nullptr; }
    RC(upload(c, &b->pan, v->post_attention_norm, bytes));
  }
  if (v->post_feedforward_norm) {
    if (b->pfn) { cudaFree(b->pfn); b->pfn = nullptr; }
    RC(upload(c, &b->pfn, v->post_feedforward_norm, bytes));
  }
  b->window = v->sliding_window;
  b->use_rope = v->use_rope != 0;
  return pipe_mark(c);
}

// ------------------------------------------------------------------------------------------ cache
extern "C" int cake_b200_cache_create(cake_b200_ctx *c, int batch, int max_seq, cake_b200_cache **out) {
  if (!c || !out || batch < 1 || max_seq < 1) return fail(CAKE_B200_EINVAL, "bad cache arguments");
  if (max_seq > c->cfg.max_seq) return fail(CAKE_B200_EINVAL, "cache max_seq %d exceeds config max_seq %d (RoPE table rows)", max_seq, c->cfg.max_seq);
  CU(cudaSetDevice(c->device));
  auto *k = new cake_b200_cache{c, batch, max_seq, c->device};
  k->gen = g_cache_gen.fetch_add(1);
  const int slots = c->cfg.layer_list ? 2 * c->cfg.n_layers : c->cfg.n_layers;  // a side mixer's entries follow the main ones
  k->k.assign(slots, nullptr);
  k->v.assign(slots, nullptr);
  k->len.assign(c->cfg.n_layers, 0);
  k->kv_heads.assign(slots, 0);
  k->kv_hd.assign(slots, 0);
  k->rec_aux.assign(slots, nullptr);
  k->vt.assign(slots, nullptr);
  k->canon_hist.assign(c->cfg.n_layers, nullptr);
  k->last_tok.assign(batch, 0);
  k->shift_state[0].assign(c->cfg.n_layers, nullptr);
  k->shift_state[1].assign(c->cfg.n_layers, nullptr);
  k->shift_cur.assign(c->cfg.n_layers, 0);
  k->rec_state.assign(slots, nullptr);
  k->conv_hist.assign(slots, nullptr);
  cudaError_t e = cudaMalloc(&k->d_pos, 4);
  if (e == cudaSuccess) e = cudaMemset(k->d_pos, 0, 4);
  if (e != cudaSuccess) {
    if (k->d_pos) cudaFree(k->d_pos);
    delete k;
    (void)cudaGetLastError();
    return fail(CAKE_B200_ECUDA, "cache_create: %s", cudaGetErrorString(e));
  }
  *out = k;
  return CAKE_B200_OK;
}
static int cache_ensure(cake_b200_cache *k, int layer) {
  if (layer < 0 || layer >= (int)k->k.size()) return fail(CAKE_B200_EINVAL, "block_idx %d out of range", layer);
  if (k->k[layer]) return CAKE_B200_OK;
  const size_t bytes = (size_t)k->batch * k->ctx->cfg.n_kv_heads * k->cap * k->ctx->cfg.head_dim * k->ctx->es;
  CU(cudaMalloc(&k->k[layer], bytes + 16));
  CU(cudaMalloc(&k->v[layer], bytes + 16));
  return CAKE_B200_OK;
}
extern "C" int cake_b200_cache_clear(cake_b200_cache *k) {
  if (!k) return fail(CAKE_B200_EINVAL, "null argument");
  for (auto &l : k->len) l = 0;
  k->embed_len = 0;  // recurrent state, histories and the previous token are ignored at position 0: nothing to wipe
  return CAKE_B200_OK;
}
extern "C" void cake_b200_cache_free(cake_b200_cache *k) {
  if (!k) return;
  cudaSetDevice(k->device);
  {  // drop everything in the ctx that points into this cache: the cached layer table and the decode graph
    std::lock_guard<std::mutex> lk(g_live_mu);
    if (g_live_ctx.count(k->ctx)) {
      cake_b200_ctx *c = k->ctx;
      cudaStreamSynchronize(c->stream);
      c->mk_sig.clear();
      if (c->g_cache == k) {
        if (c->gexec) { cudaGraphExecDestroy(c->gexec); c->gexec = nullptr; }
        if (c->graph) { cudaGraphDestroy(c->graph); c->graph = nullptr; }
        c->g_cache = nullptr;
        c->g_block_idx.clear();
      }
    }
  }
  for (void *p : k->k)
    if (p) cudaFree(p);
  for (void *p : k->v)
    if (p) cudaFree(p);
  for (auto &v : k->shift_state)
    for (float *p : v)
      if (p) cudaFree(p);
  for (float *p : k->rec_state)
    if (p) cudaFree(p);
  for (void *p : k->conv_hist)
    if (p) cudaFree(p);
  for (float *p : k->rec_aux)
    if (p) cudaFree(p);
  for (void *p : k->vt)
    if (p) cudaFree(p);
  for (float *p : k->canon_hist)
    if (p) cudaFree(p);
  cudaFree(k->d_pos);
  (void)cudaGetLastError();
  delete k;
}
extern "C" int cake_b200_cache_len(const cake_b200_cache *k, int block_idx) {
  if (!k || block_idx < 0 || block_idx >= (int)k->len.size()) return -1;
  return k->len[block_idx];
}
extern "C" int cake_b200_cache_read(cake_b200_cache *k, int block_idx, int which, void *out_host, size_t bytes) {
  if (!k || !out_host) return fail(CAKE_B200_EINVAL, "null argument");
  cake_b200_ctx *c = k->ctx;
  CU(cudaSetDevice(c->device));
  if (block_idx < 0 || block_idx >= (int)k->len.size() || !k->k[block_idx]) return fail(CAKE_B200_EINVAL, "layer %d has no cache", block_idx);
  const int len = k->len[block_idx];
  const int hd = k->kv_hd[block_idx] ? k->kv_hd[block_idx] : c->cfg.head_dim, nkv = k->kv_heads[block_idx] ? k->kv_heads[block_idx] : c->cfg.n_kv_heads;
  if (which && !k->v[block_idx]) return fail(CAKE_B200_EINVAL, "layer %d keeps no V cache (its values are its keys)", block_idx);
  const size_t need = (size_t)k->batch * nkv * len * hd * c->es;
  if (bytes < need) return fail(CAKE_B200_EINVAL, "cache_read needs %zu bytes", need);
  CU(cudaStreamSynchronize(c->stream));
  const char *src = (const char *)(which ? k->v[block_idx] : k->k[block_idx]);
  CU(cudaMemcpy2D(out_host, (size_t)len * hd * c->es, src, (size_t)k->cap * hd * c->es, (size_t)len * hd * c->es,
                  (size_t)k->batch * nkv, cudaMemcpyDeviceToHost));
  return CAKE_B200_OK;
}
extern "C" int cake_b200_cache_fill_synthetic(cake_b200_cache *k, const int *block_idx, int n_blocks, int len,
                                              uint32_t seed) {
  if (!k || (!block_idx && n_blocks > 0) || n_blocks < 0 || len < 0) return fail(CAKE_B200_EINVAL, "bad cache_fill_synthetic arguments");
  cake_b200_ctx *c = k->ctx;
  CU(cudaSetDevice(c->device));
  if (len > k->cap) return fail(CAKE_B200_EINVAL, "len %d > cache capacity %d", len, k->cap);
  if (c->cfg.layer_list) return fail(CAKE_B200_EINVAL, "cache_fill_synthetic is for the Llama-family blocks");
  for (int i = 0; i < n_blocks; i++) {
    const int l = block_idx[i];
    RC(cache_ensure(k, l));
    const size_t n = (size_t)k->batch * c->cfg.n_kv_heads * k->cap * c->cfg.head_dim;
    RC(DISPATCH_T(c->cfg.dtype, T_LAMBDA {
      typedef typename decltype(tag_)::type T;
      fill_synth_kernel<T><<<1024, 256, 0, c->stream>>>((T *)k->k[l], n, seed + 2 * l, 1.0f);
      fill_synth_kernel<T><<<1024, 256, 0, c->stream>>>((T *)k->v[l], n, seed + 2 * l + 1, 1.0f);
      return CAKE_B200_OK;
    }));
    k->len[l] = len;
  }
  CU(cudaGetLastError());
  return CAKE_B200_OK;
}

// ------------------------------------------------------------------------------------------ decode path (batch 1, seq 1)
// x_in -> x_out through `n` blocks; position comes from cache->d_pos (device).  5 kernels per layer.
static int enqueue_qkv(cake_b200_ctx *c, const cake_b200_block *b, const void *x) {
  // rms_1 + fused qkv projection (+bias)                           transformer.rs:112, attention.rs:162-164
  GemvArgs a{};
  a.W = b->wqkv; a.x = x; a.norm_w = b->ln1; a.bias = b->bqkv; a.out = c->qkv; a.eps = c->cfg.rms_eps;
  a.N = c->nqkv; a.K = c->cfg.hidden;
  return launch_gemv<EPI_PLAIN>(c, a);
}
static int enqueue_attn(cake_b200_ctx *c, const cake_b200_block *b, cake_b200_cache *kc, int l) {
  // qk-norm, RoPE, KV append, GQA attention                        attention.rs:202-346, cache.rs:184-210
  const cake_b200_config &f = c->cfg;
  AttnDecodeArgs a{};
  a.qkv = c->qkv; a.kcache = kc->k[l]; a.vcache = kc->v[l]; a.cos_t = c->cos_t; a.sin_t = c->sin_t;
  a.q_norm = b->qn; a.k_norm = b->kn; a.y = c->y; a.ws_ml = c->ws_ml; a.ws_acc = c->ws_acc;
  a.counters = c->attn_counters; a.d_pos = kc->d_pos; a.n_heads = f.n_heads; a.n_kv = f.n_kv_heads;
  a.cap = kc->cap; a.rot = c->rot; a.nsplit = c->nsplit; a.eps = f.rms_eps;
  a.scale = (float)(1.0 / sqrt((double)f.head_dim));
  a.window = f.sliding_window;
  dim3 grid(c->nsplit, f.n_kv_heads), block(ATTN_THREADS);
  const size_t smem = attn_smem_bytes(f.head_dim, c->es);
  return DISPATCH_T(f.dtype, T_LAMBDA {
    typedef typename decltype(tag_)::type T;
    switch (f.head_dim) {
      case 16: return launch_pdl(c, attn_decode_kernel<T, 16>, grid, block, smem, a);
      case 32: return launch_pdl(c, attn_decode_kernel<T, 32>, grid, block, smem, a);
      case 64: return launch_pdl(c, attn_decode_kernel<T, 64>, grid, block, smem, a);
      case 128: return launch_pdl(c, attn_decode_kernel<T, 128>, grid, block, smem, a);
      default: return launch_pdl(c, attn_decode_kernel<T, 256>, grid, block, smem, a);
    }
  });
}
static int enqueue_oproj(cake_b200_ctx *c, const cake_b200_block *b, const void *residual, void *out) {
  // o_proj + residual                                              attention.rs:354, transformer.rs:123
  GemvArgs a{};
  a.W = b->wo; a.x = c->y; a.residual = residual; a.out = out; a.N = c->cfg.hidden;
  a.K = c->cfg.n_heads * c->cfg.head_dim;
  return launch_gemv<EPI_RESIDUAL>(c, a);
}
static int enqueue_gate_up(cake_b200_ctx *c, const cake_b200_block *b, const void *x1) {
  // rms_2 + gate_up + silu*mul                                     transformer.rs:129, mlp.rs:22-28
  GemvArgs a{};
  a.W = b->wgu; a.x = x1; a.norm_w = b->ln2; a.out = c->mm; a.eps = c->cfg.rms_eps; a.N = 2 * c->cfg.inter; a.act = c->cfg.use_gelu_mlp ? 1 : 0;
  a.K = c->cfg.hidden;
  return launch_gemv<EPI_SWIGLU>(c, a);
}
static int enqueue_down(cake_b200_ctx *c, const cake_b200_block *b, const void *residual, void *out) {
  // down + residual                                                mlp.rs:30, transformer.rs:131
  GemvArgs a{};
  a.W = b->wd; a.x = c->mm; a.residual = residual; a.out = out; a.N = c->cfg.hidden; a.K = c->cfg.inter;
  return launch_gemv<EPI_RESIDUAL>(c, a);
}

static int enqueue_decode_layers(cake_b200_ctx *c, cake_b200_block *const *blocks, const int *block_idx, int n,
                                 cake_b200_cache *kc, const void *x_in, void *x_out) {
  const void *cur = x_in;
  for (int i = 0; i < n; i++) {
    const cake_b200_block *b = blocks[i];
    void *dst = (i == n - 1) ? x_out : c->xa;
    RC(enqueue_qkv(c, b, cur));
    RC(enqueue_attn(c, b, kc, block_idx[i]));
    RC(enqueue_oproj(c, b, cur, c->xb));
    RC(enqueue_gate_up(c, b, c->xb));
    RC(enqueue_down(c, b, c->xb, dst));
    cur = dst;
  }
  return CAKE_B200_OK;
}

// ------------------------------------------------------------------------------------------ megakernel plan + launch
static int plan_mk_geom(const cake_b200_ctx *c, int N, int K, int G, MkGeom *g, int *partial_floats, int *max_groups) {
  const int es = c->es;
  if (K % 64 != 0 || N % G != 0) return fail(CAKE_B200_EINVAL, "mega: K=%d must be a multiple of 64, N=%d of %d", K, N, G);
  int KC = K;
  while ((size_t)KC * es > MK_STAGE_BYTES && (KC / 2) % 64 == 0) KC /= 2;
  const size_t seg = (size_t)KC * es;
  if (seg > MK_STAGE_BYTES) return fail(CAKE_B200_EINVAL, "mega: K=%d cannot be staged", K);
  int RS = 1;
  while (RS < 64 && (size_t)(RS * 2) * seg <= MK_STAGE_BYTES) RS *= 2;
  int WPR, RPW;
  if (RS >= MK_CW) { WPR = 1; RPW = RS / MK_CW; }
  else { WPR = MK_CW / RS; RPW = 1; }
  while (WPR > 1 && ((KC / 8) % WPR != 0)) { WPR /= 2; }  // slices must divide the segment's 16-byte vectors
  if (RS * RPW < (MK_CW / WPR) * RPW || RS != (MK_CW / WPR) * RPW)  // every row slot must map to a staged row
    return fail(CAKE_B200_EINVAL, "mega: unsupported geometry N=%d K=%d (KC=%d RS=%d WPR=%d)", N, K, KC, RS, WPR);
  *g = MkGeom{N, K, KC, RS, WPR, RPW};
  // per-CTA cap of row groups in one phase: twice the even share (dynamic claiming, decode_mega.cuh mk_split)
  const int n_groups = (N + RS - 1) / RS;
  const int cap = 2 * ((n_groups + c->sm_count - 1) / c->sm_count) + 4;
  if (cap > *max_groups) *max_groups = cap;
  // *partial_floats collects max(RS*WPR) here and the static-path need; plan_mega multiplies by the global cap
  if (RS * WPR > *partial_floats % 65536) *partial_floats = (*partial_floats / 65536) * 65536 + RS * WPR;
  const int pf_static = (((N / G) / c->sm_count) + 1) * G * WPR;
  if (pf_static > *partial_floats / 65536) *partial_floats = pf_static * 65536 + *partial_floats % 65536;
  return CAKE_B200_OK;
}

struct MkPlan {
  MkArgs a;
  size_t smem;
};
static bool mega_supported(const cake_b200_ctx *c) {
  const int G = c->cfg.n_heads / c->cfg.n_kv_heads;
#define MK_CASE(HD_, G_) if (c->cfg.head_dim == HD_ && G == G_) return true;
  MK_FOR_ALL(MK_CASE)
#undef MK_CASE
  return false;
}
static int plan_mega(cake_b200_ctx *c, cake_b200_cache *kc, bool with_head, MkPlan *p) {
  const cake_b200_config &f = c->cfg;
  MkArgs &a = p->a;
  memset(&a, 0, sizeof(a));
  int pf = 0, mg = 0;
  RC(plan_mk_geom(c, c->nqkv, f.hidden, 1, &a.g_qkv, &pf, &mg));
  RC(plan_mk_geom(c, f.hidden, f.n_heads * f.head_dim, 1, &a.g_o, &pf, &mg));
  RC(plan_mk_geom(c, 2 * f.inter, f.hidden, 2, &a.g_gu, &pf, &mg));
  RC(plan_mk_geom(c, f.hidden, f.inter, 1, &a.g_down, &pf, &mg));
  if (with_head) RC(plan_mk_geom(c, f.vocab, f.hidden, 1, &a.g_head, &pf, &mg));
  {  // partial-sum scratch: every phase may use up to `mg` groups of its own RS*WPR floats (dynamic), or its static rows
    const int dyn_need = mg * (pf % 65536), static_need = pf / 65536;
    pf = dyn_need > static_need ? dyn_need : static_need;
  }
  a.partial_floats = pf;
  a.max_groups = mg;
  a.tickets = c->tickets;
  {
    const char *e = getenv("CAKE_B200_L2_PREFETCH");
    a.l2_prefetch = (e && e[0] >= '1' && e[0] <= '2') ? e[0] - '0' : 0;
  }
  a.hidden = f.hidden; a.inter = f.inter; a.n_heads = f.n_heads; a.n_kv = f.n_kv_heads; a.hd = f.head_dim;
  a.rot = c->rot; a.cap = kc ? kc->cap : 0; a.nsplit = c->nsplit; a.eps = f.rms_eps;
  a.scale = (float)(1.0 / sqrt((double)f.head_dim));
  a.max_k = f.inter > f.hidden ? f.inter : f.hidden;
  if (f.n_heads * f.head_dim > a.max_k) a.max_k = f.n_heads * f.head_dim;
  a.xa = c->xa; a.xb = c->xb; a.qkv = c->qkv; a.y = c->y; a.mm = c->mm;
  a.ws_ml = c->ws_ml; a.ws_acc = c->ws_acc; a.attn_counters = c->attn_counters;
  a.cos_t = c->cos_t; a.sin_t = c->sin_t; a.d_pos = kc ? kc->d_pos : nullptr; a.d_step = c->d_step; a.gbar = c->gbar;
  a.vocab = f.vocab; a.embed = c->embed; a.d_token = c->d_token;
  a.ln_f = c->ln_f; a.lm_head = c->lm_head; a.logits = c->logits; a.part_val = c->part_val; a.part_idx = c->part_idx;
  a.argmax_counter = c->argmax_counter; a.token_out = c->d_token; a.token_ring = nullptr; a.ring_cap = TOKEN_RING;
  a.trace = c->trace;
  a.step_trace = c->step_trace;
  a.trace_tag = 0;
  a.act = f.use_gelu_mlp ? 1 : 0;
  a.window = f.sliding_window;
  int ns = MK_MAX_STAGES;
  const size_t limit = 227 * 1024 - 4096;  // the kernel also has ~2.2 KB of static shared memory
  while (ns > 2 && mk_smem_bytes(a.max_k, pf, mg, ns, c->es) > limit) ns--;
  a.n_stages = ns;
  p->smem = mk_smem_bytes(a.max_k, pf, mg, ns, c->es);
  if (p->smem > limit) return fail(CAKE_B200_EINVAL, "mega: needs %zu B of shared memory", p->smem);
  return CAKE_B200_OK;
}

template <typename T> static int launch_mega_T(cake_b200_ctx *c, cudaLaunchConfig_t *cfg, const MkArgs &a) {
  const int G = c->cfg.n_heads / c->cfg.n_kv_heads;
#define MK_CASE(HD_, G_)                                                \
  if (c->cfg.head_dim == HD_ && G == G_) {                              \
    CU(cudaLaunchKernelEx(cfg, decode_mega_kernel<T, HD_, G_>, a));     \
    return CAKE_B200_OK;                                                \
  }
  MK_FOR_ALL(MK_CASE)
#undef MK_CASE
  return fail(CAKE_B200_EINVAL, "megakernel: head_dim %d with %d query heads per kv head is not instantiated", c->cfg.head_dim, G);
}

static int launch_mega(cake_b200_ctx *c, const MkPlan &p) {
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(c->sm_count);
  cfg.blockDim = dim3(MK_THREADS);
  cfg.dynamicSmemBytes = p.smem;
  cfg.stream = c->stream;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeCooperative;  // all CTAs must be co-resident (grid barriers inside)
  at[0].val.cooperative = 1;
  cfg.attrs = at;
  cfg.numAttrs = 1;
  const MkArgs &a = p.a;
  CU(cudaMemsetAsync(c->tickets, 0, sizeof(unsigned) * (4 * (size_t)a.n_layers + 4), c->stream));  // a memset node in the graph
  int rc = DISPATCH_T(c->cfg.dtype, T_LAMBDA {
    typedef typename decltype(tag_)::type T;
    return launch_mega_T<T>(c, &cfg, a);
  });
  RC(rc);
  if (c->capturing) c->g_kernels++;
  else c->launches++;
  return CAKE_B200_OK;
}

static void fill_mk_table(MkLayer *tab, cake_b200_block *const *blocks, const int *block_idx, int n, cake_b200_cache *kc) {
  for (int i = 0; i < n; i++) {
    const cake_b200_block *b = blocks[i];
    tab[i] = MkLayer{b->wqkv, b->wo, b->wgu, b->wd, b->ln1, b->ln2, b->bqkv, b->qn, b->kn, kc->k[block_idx[i]], kc->v[block_idx[i]]};
  }
}

// x_in -> x_out through n blocks in ONE persistent kernel; position from cache->d_pos
static int enqueue_mega_layers(cake_b200_ctx *c, cake_b200_block *const *blocks, const int *block_idx, int n,
                               cake_b200_cache *kc, const void *x_in, void *x_out) {
  if (n > MK_MAX_LAYERS) return fail(CAKE_B200_EINVAL, "more than %d blocks in one call", MK_MAX_LAYERS);
  std::vector<const void *> sig;
  sig.push_back(kc);
  sig.push_back(reinterpret_cast<const void *>((uintptr_t)kc->gen));
  for (int i = 0; i < n; i++) { sig.push_back(blocks[i]); sig.push_back(kc->k[block_idx[i]]); sig.push_back(kc->v[block_idx[i]]); }
  if (sig != c->mk_sig) {  // (re)build the layer table; rare
    CU(cudaStreamSynchronize(c->stream));
    fill_mk_table(c->mk_tab_host, blocks, block_idx, n, kc);
    CU(cudaMemcpyAsync(c->mk_tab_dev, c->mk_tab_host, sizeof(MkLayer) * n, cudaMemcpyHostToDevice, c->stream));
    c->mk_sig = sig;
  }
  MkPlan p;
  RC(plan_mega(c, kc, false, &p));
  p.a.layers = c->mk_tab_dev;
  p.a.n_layers = n;
  p.a.x_in = x_in;
  p.a.x_out = x_out;
  p.a.has_head = 0;
  p.a.advance = 0;
  return launch_mega(c, p);
}

// ln_f + lm_head + greedy argmax on one hidden row -> logits_out (nullable), token -> c->d_token
static int enqueue_head(cake_b200_ctx *c, const void *x_row, void *logits_out, bool ring) {
  GemvArgs a{};
  a.W = c->lm_head; a.x = x_row; a.norm_w = c->ln_f; a.out = logits_out; a.eps = c->cfg.rms_eps;
  a.N = c->cfg.vocab; a.K = c->cfg.hidden;
  a.part_val = c->part_val; a.part_idx = c->part_idx; a.counter = c->argmax_counter; a.token_out = c->d_token;
  a.token_ring = ring ? c->token_ring : nullptr; a.step = c->d_step; a.ring_cap = TOKEN_RING;
  return launch_gemv<EPI_ARGMAX>(c, a);
}

// ------------------------------------------------------------------------------------------ TMA tensor maps (driver entry point, no -lcuda)
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                                  const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn g_encode_tiled = nullptr;
static int tmap_init() {
  if (g_encode_tiled) return CAKE_B200_OK;
  void *fn = nullptr;
  cudaDriverEntryPointQueryResult q;
  CU(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q));
  if (!fn || q != cudaDriverEntryPointSuccess) return fail(CAKE_B200_ECUDA, "cuTensorMapEncodeTiled is not available from this driver");
  g_encode_tiled = (EncodeTiledFn)fn;
  return CAKE_B200_OK;
}
// [rows, K] row-major matrix of D -> 2-D map with a (64 x box_rows) box and 128-byte swizzle
// K: the visible columns (the TMA unit zero-fills past them); ld: the row stride in elements when it is not K
static int make_tmap(CUtensorMap *m, const void *ptr, uint64_t rows, uint64_t K, int dtype, uint32_t box_rows, uint64_t ld = 0) {
  RC(tmap_init());
  const cuuint64_t gdim[2] = {K, rows};
  const cuuint64_t gstride[1] = {(ld ? ld : K) * 2};
  const cuuint32_t box[2] = {(cuuint32_t)TC_BK, box_rows};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult r = g_encode_tiled(m, dtype == CAKE_B200_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2,
                                    const_cast<void *>(ptr), gdim, gstride, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                    CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(CAKE_B200_ECUDA, "cuTensorMapEncodeTiled(rows=%llu, K=%llu) -> CUresult %d", (unsigned long long)rows, (unsigned long long)K, (int)r);
  return CAKE_B200_OK;
}

// [slabs][rows][cols] tensor of D with a slab stride of slab_rows rows -> 3-D map, (64 x box_rows x 1) box, 128-byte swizzle.
// `rows` is the VISIBLE extent: the TMA unit zero-fills rows past it (query rows >= S, keys >= the attended length), so a
// tile never carries a neighbouring slab's rows or uninitialised cache memory into an MMA.
// slab_stride_elems > 0: the slabs lie that many elements apart (heads side by side inside a row) instead of slab_rows rows.
static int make_tmap3(CUtensorMap *m, const void *ptr, uint64_t cols, uint64_t row_stride_elems, uint64_t rows, uint64_t slab_rows,
                      uint64_t slabs, int dtype, uint32_t box_rows, uint64_t slab_stride_elems = 0) {
  RC(tmap_init());
  const cuuint64_t gdim[3] = {cols, rows, slabs};
  const cuuint64_t gstride[2] = {row_stride_elems * 2, (slab_stride_elems ? slab_stride_elems : slab_rows * row_stride_elems) * 2};
  const cuuint32_t box[3] = {64u, box_rows, 1u};
  const cuuint32_t estr[3] = {1, 1, 1};
  const CUresult r = g_encode_tiled(m, dtype == CAKE_B200_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3,
                                    const_cast<void *>(ptr), gdim, gstride, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                    CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(CAKE_B200_ECUDA, "cuTensorMapEncodeTiled(3d: cols=%llu rows=%llu slabs=%llu) -> CUresult %d", (unsigned long long)cols, (unsigned long long)rows, (unsigned long long)slabs, (int)r);
  return CAKE_B200_OK;
}

static bool tc_gemm_ok(int M, int N, int K) { return M >= 1 && N % TC_BN == 0 && K % TC_BK == 0; }

// C = epi(A[M,K] W[N,K]^T) on the tensor cores (gemm_tc.cuh)
struct TcExtra {  // optional modes of the tensor-core GEMM (TcParams in gemm_tc.cuh)
  const int *tile_group = nullptr;  // grouped product: W holds n_groups stacked [N, K] matrices
  int n_groups = 1;
  const float *row_scale = nullptr;
  int b_kwrap = 0, w_cols = 0, w_ld = 0;  // W's k coordinate wraps at b_kwrap; its visible columns / row stride when not K
  int w_rows = 0;                         // W's visible rows when fewer than N (the rest reads as zeros)
  int a_ld = 0;                           // A's row stride in elements when it is a column range of a wider buffer
};
template <typename T, int EPI>
static int gemm_tc_T(cake_b200_ctx *c, const void *A, const void *W, const void *bias, const void *res, void *C, int M, int N, int K,
                     int act = -1, int ldc = 0, float cap = 0.f, const TcExtra &x = TcExtra{}) {
  // 128 x 256 tiles when N allows and there are enough tiles to fill the chip; CAKE_B200_TC_BN=128 forces the small tile (A/B aid)
  static const int force_bn = []() { const char *e = getenv("CAKE_B200_TC_BN"); return e ? atoi(e) : 0; }();
  const int tiles_m = (M + TC_BM - 1) / TC_BM;
  const bool big = force_bn ? force_bn == 256 && N % 256 == 0 : (N % 256 == 0 && tiles_m * (N / 256) >= c->sm_count);
  const int bn = big ? 256 : 128;
  // pairs of CTAs sharing the W tile by TMA multicast (gemm_tc.cuh MC): needs an even number of 128-row tiles
  static const int no_mc = []() { const char *e = getenv("CAKE_B200_TC_MC"); return (e && e[0] == '0') ? 1 : 0; }();
  const bool mc = big && !no_mc && M % 256 == 0 && (tiles_m / 2) * (N / 256) >= c->sm_count / 2 && !x.tile_group && !x.b_kwrap;
  CUtensorMap ma, mb;
  RC(make_tmap(&ma, A, (uint64_t)M, (uint64_t)K, c->cfg.dtype, TC_BM, (uint64_t)x.a_ld));
  RC(make_tmap(&mb, W, x.w_rows ? (uint64_t)x.w_rows : (uint64_t)N * x.n_groups, (uint64_t)(x.w_cols ? x.w_cols : K), c->cfg.dtype,
               mc ? 128u : (uint32_t)bn, (uint64_t)x.w_ld ? (uint64_t)x.w_ld : (uint64_t)K));
  TcParams p{bias, res, C, M, N, K, act >= 0 ? act : (c->cfg.use_gelu_mlp ? 1 : 0), ldc, cap, x.tile_group, x.row_scale, x.b_kwrap};
  const int tiles = tiles_m * (N / bn);
  dim3 grid(tiles < c->sm_count ? tiles : c->sm_count), block(TC_THREADS);
  if (mc) {
    dim3 g2((unsigned)(c->sm_count & ~1));
    return launch_cluster_pdl(c, gemm_tc_kernel<T, EPI, 256, true>, g2, block, (size_t)TcCfg<256>::SMEM_BYTES, 2u, ma, mb, p);
  }
  if (big) return launch_pdl(c, gemm_tc_kernel<T, EPI, 256>, grid, block, (size_t)TcCfg<256>::SMEM_BYTES, ma, mb, p);
  return launch_pdl(c, gemm_tc_kernel<T, EPI, 128>, grid, block, (size_t)TcCfg<128>::SMEM_BYTES, ma, mb, p);
}

// ------------------------------------------------------------------------------------------ prefill path (any batch / seq)
static int pf_reserve(cake_b200_ctx *c, size_t rows) {
  if (rows <= c->pf_rows) return CAKE_B200_OK;
  CU(cudaStreamSynchronize(c->stream));
  void **bufs[] = {&c->pf_h, &c->pf_qkv, &c->pf_y, &c->pf_x1, &c->pf_gu, &c->pf_mm};
  for (void **b : bufs)
    if (*b) { cudaFree(*b); *b = nullptr; }
  const cake_b200_config &f = c->cfg;
  const size_t es = c->es;
  CU(cudaMalloc(&c->pf_h, rows * f.hidden * es));
  CU(cudaMalloc(&c->pf_qkv, rows * c->nqkv * es));
  CU(cudaMalloc(&c->pf_y, rows * f.n_heads * f.head_dim * es));
  CU(cudaMalloc(&c->pf_x1, rows * f.hidden * es));
  CU(cudaMalloc(&c->pf_gu, rows * 2 * f.inter * es));
  CU(cudaMalloc(&c->pf_mm, rows * f.inter * es));
  c->pf_rows = rows;
  return CAKE_B200_OK;
}

// RMSNorm over M rows of n: warp-per-row vector kernel for n = 256 * {4, 8, 16, 32} and 16-byte aligned rows, else the generic one
template <typename T>
static int rmsnorm_rows_T(cake_b200_ctx *c, const void *x, const void *w, void *out, int M, int n, float eps) {
  const bool al = (((uintptr_t)x | (uintptr_t)w | (uintptr_t)out) & 15) == 0;
  const dim3 g((unsigned)((M + 7) / 8)), blk(256);
  if (al && n == 1024) return launch_pdl(c, rmsnorm_rows_vec_kernel<T, 4>, g, blk, 0, (const T *)x, (const T *)w, (T *)out, M, eps);
  if (al && n == 2048) return launch_pdl(c, rmsnorm_rows_vec_kernel<T, 8>, g, blk, 0, (const T *)x, (const T *)w, (T *)out, M, eps);
  if (al && n == 4096) return launch_pdl(c, rmsnorm_rows_vec_kernel<T, 16>, g, blk, 0, (const T *)x, (const T *)w, (T *)out, M, eps);
  if (al && n == 8192) return launch_pdl(c, rmsnorm_rows_vec_kernel<T, 32>, g, blk, 0, (const T *)x, (const T *)w, (T *)out, M, eps);
  return launch_pdl(c, rmsnorm_rows_kernel<T>, dim3(M), dim3(256), 0, (const T *)x, (const T *)w, (T *)out, n, eps);
}

template <typename T>
static int gemm_T(cake_b200_ctx *c, const void *A, const void *W, const void *bias, const void *res, void *C, int M,
                  int N, int K) {
  dim3 grid((N + GV0_BN - 1) / GV0_BN, (M + GV0_BM - 1) / GV0_BM), block(256);
  return launch_pdl(c, gemm_v0_kernel<T>, grid, block, 0, (const T *)A, (const T *)W, (const T *)bias, (const T *)res,
                    (T *)C, M, N, K);
}

static int enqueue_prefill_layers(cake_b200_ctx *c, cake_b200_block *const *blocks, const int *block_idx, int n,
                                  cake_b200_cache *kc, const void *x_in, void *x_out, int B, int S, int pos0) {
  const cake_b200_config &f = c->cfg;
  const int H = f.hidden, I = f.inter, hd = f.head_dim, sq = f.n_heads * hd, M = B * S;
  RC(pf_reserve(c, (size_t)M));
  // cache.rs:173-205: a call on a non-empty cache sees the last `window` positions of cat(cache, new) — every query of
  // the chunk the same old rows [ws, pos0) — while the first call (pos0 == 0) attends over everything it stores.  The
  // attention kernels only see row indices relative to ws (base pointers advanced by ws rows); K/V append is unaffected.
  // per block (attention.rs load_custom gives every layer its own window): block_window() below
  auto block_window = [&](const cake_b200_block *b, int *ws_out) -> int {
    const int w = b->window >= 0 ? b->window : f.sliding_window;
    int ws = 0;
    if (w > 0 && pos0 > 0 && pos0 + S > w) {
      ws = pos0 + S - w;
      if (ws > pos0) return fail(CAKE_B200_EINVAL, "a chunk of %d tokens on a non-empty cache exceeds the sliding window %d", S, w);
    }
    *ws_out = ws;
    return CAKE_B200_OK;
  };
  for (int i = 0; i < n; i++) { int t; RC(block_window(blocks[i], &t)); }  // refuse before anything is enqueued
  const char *env_tc = getenv("CAKE_B200_NO_TC");
  const bool use_tc = !(env_tc && env_tc[0] == '1');  // CAKE_B200_NO_TC=1: CUDA-core GEMM (A/B testing aid)
  return DISPATCH_T(f.dtype, T_LAMBDA {
      typedef typename decltype(tag_)::type T;
    const void *cur = x_in;
    for (int i = 0; i < n; i++) {
      const cake_b200_block *b = blocks[i];
      const int l = block_idx[i];
      int ws = 0;
      RC(block_window(b, &ws));
      const size_t wsoff = (size_t)ws * hd;
      const int apos0 = pos0 - ws;
      // transformer.rs:112 rms_1 — or none: olmo2/block.rs:70 feeds x itself to the attention
      const void *att_in = cur;
      if (b->ln1) { RC(rmsnorm_rows_T<T>(c, cur, b->ln1, c->pf_h, M, H, f.rms_eps)); att_in = c->pf_h; }
      if (use_tc && tc_gemm_ok(M, c->nqkv, H) && ((uintptr_t)att_in & 15) == 0) RC((gemm_tc_T<T, TCE_PLAIN>(c, att_in, b->wqkv, b->bqkv, nullptr, c->pf_qkv, M, c->nqkv, H)));
      else RC(gemm_T<T>(c, att_in, b->wqkv, b->bqkv, nullptr, c->pf_qkv, M, c->nqkv, H));
      const void *qn = b->qn, *kn = b->kn;
      if (f.pre_reshape_qk_norm && qn && kn) {  // attention.rs:176-192: RmsNorm over the whole q and k projections, in place
        RC(launch_pdl(c, rmsnorm_strided_kernel<T>, dim3(M), dim3(256), 0, (T *)c->pf_qkv, (const T *)qn, c->nqkv, sq, f.rms_eps));
        RC(launch_pdl(c, rmsnorm_strided_kernel<T>, dim3(M), dim3(256), 0, (T *)c->pf_qkv + sq, (const T *)kn, c->nqkv, (int)(f.n_kv_heads * hd), f.rms_eps));
        qn = kn = nullptr;
      }
      const int rope_on = b->use_rope ? 1 : 0;
      {
        const long items = (long)M * (f.n_heads + 2 * f.n_kv_heads);
        if (hd == 128 && c->rot == 128 && ((uintptr_t)c->cos_t & 3) == 0)  // full rotary on 128-wide heads: token-per-warp vector kernel
          RC(launch_pdl(c, rope_append_vec_kernel<T>, dim3((unsigned)((M + 3) / 4)), dim3(128), 0, (T *)c->pf_qkv, (T *)kc->k[l], (T *)kc->v[l],
                        (const T *)c->cos_t, (const T *)c->sin_t, (const T *)qn, (const T *)kn, B, S, f.n_heads, f.n_kv_heads, kc->cap, pos0,
                        f.rms_eps, rope_on));
        else
        RC(launch_pdl(c, rope_append_kernel<T>, dim3((unsigned)((items + 3) / 4)), dim3(128), (size_t)4 * hd * 4,
                      (T *)c->pf_qkv, (T *)kc->k[l], (T *)kc->v[l], (const T *)c->cos_t, (const T *)c->sin_t,
                      (const T *)qn, (const T *)kn, B, S, f.n_heads, f.n_kv_heads, hd, c->rot, kc->cap, pos0, f.rms_eps, rope_on));
      }
      if (use_tc && (hd == 64 || hd == 128)) {  // tensor-core flash attention (attn_prefill.cuh)
        dim3 grid((S + FA_BM - 1) / FA_BM, f.n_heads, B), block(FA_THREADS);
        const float sc = (float)(1.0 / sqrt((double)hd));
        // head_dim 128: tcgen05 flash attention (attn_prefill_tc.cuh); CAKE_B200_FA=mma keeps the mma.sync kernel (A/B aid)
        static const bool fa_mma = []() { const char *e = getenv("CAKE_B200_FA"); return e && !strcmp(e, "mma"); }();
        static const float fa_tau = []() { const char *e = getenv("CAKE_B200_FA_TAU"); return e ? (float)atof(e) : 5.545f; }();
        if (hd == 128 && !fa_mma) {
          CUtensorMap mq, mk, mv;
          const uint64_t nqkv_cols = (uint64_t)(f.n_heads + 2 * f.n_kv_heads) * hd;
          RC(make_tmap3(&mq, c->pf_qkv, nqkv_cols, nqkv_cols, (uint64_t)S, (uint64_t)S, (uint64_t)B, f.dtype, FT_BM));
          RC(make_tmap3(&mk, (const T *)kc->k[l] + wsoff, (uint64_t)hd, (uint64_t)hd, (uint64_t)(apos0 + S), (uint64_t)kc->cap,
                        (uint64_t)B * f.n_kv_heads, f.dtype, FT_BN));
          RC(make_tmap3(&mv, (const T *)kc->v[l] + wsoff, (uint64_t)hd, (uint64_t)hd, (uint64_t)(apos0 + S), (uint64_t)kc->cap,
                        (uint64_t)B * f.n_kv_heads, f.dtype, FT_BN));
          dim3 gt((S + FT_BM - 1) / FT_BM, f.n_heads, B);
          RC(launch_pdl(c, attn_prefill_tc_kernel<T>, gt, dim3(FT_THREADS), (size_t)FT_SMEM_BYTES, mq, mk, mv, (T *)c->pf_y, S, f.n_heads,
                        f.n_kv_heads, apos0, sc * 1.4426950408889634f, fa_tau * 1.4426950408889634f));
        } else if (hd == 128)
          RC(launch_pdl(c, attn_prefill_mma_kernel<T, 128>, grid, block, (size_t)4 * FA_BN * 128 * 2, (const T *)c->pf_qkv,
                        (const T *)kc->k[l] + wsoff, (const T *)kc->v[l] + wsoff, (T *)c->pf_y, S, f.n_heads, f.n_kv_heads, kc->cap, apos0, sc));
        else
          RC(launch_pdl(c, attn_prefill_mma_kernel<T, 64>, grid, block, (size_t)4 * FA_BN * 64 * 2, (const T *)c->pf_qkv,
                        (const T *)kc->k[l] + wsoff, (const T *)kc->v[l] + wsoff, (T *)c->pf_y, S, f.n_heads, f.n_kv_heads, kc->cap, apos0, sc));
      } else {
        const long items = (long)M * f.n_heads;
        RC(launch_pdl(c, attn_prefill_v0_kernel<T>, dim3((unsigned)((items + 3) / 4)), dim3(128), 0, (const T *)c->pf_qkv,
                      (const T *)kc->k[l] + wsoff, (const T *)kc->v[l] + wsoff, (T *)c->pf_y, B, S, f.n_heads, f.n_kv_heads, hd, kc->cap,
                      apos0, (float)(1.0 / sqrt((double)hd))));
      }
      if (b->pan) {  // olmo2/block.rs:77-79, gemma3/block.rs:120-122: x1 = x + rms_norm(o_proj(y))  (pf_h is free again here)
        if (use_tc && tc_gemm_ok(M, H, sq)) RC((gemm_tc_T<T, TCE_PLAIN>(c, c->pf_y, b->wo, nullptr, nullptr, c->pf_h, M, H, sq)));
        else RC(gemm_T<T>(c, c->pf_y, b->wo, nullptr, nullptr, c->pf_h, M, H, sq));
        RC(launch_pdl(c, rmsnorm_residual_rows_kernel<T>, dim3(M), dim3(256), 0, (const T *)c->pf_h, (const T *)b->pan, (const T *)cur, (T *)c->pf_x1, H, f.rms_eps));
      } else if (use_tc && tc_gemm_ok(M, H, sq) && ((uintptr_t)cur & 15) == 0) RC((gemm_tc_T<T, TCE_RESIDUAL>(c, c->pf_y, b->wo, nullptr, cur, c->pf_x1, M, H, sq)));
      else RC(gemm_T<T>(c, c->pf_y, b->wo, nullptr, cur, c->pf_x1, M, H, sq));
      const void *mlp_in = c->pf_x1;
      if (b->ln2) { RC(rmsnorm_rows_T<T>(c, c->pf_x1, b->ln2, c->pf_h, M, H, f.rms_eps)); mlp_in = c->pf_h; }
      if (use_tc && tc_gemm_ok(M, 2 * I, H)) {
        RC((gemm_tc_T<T, TCE_SWIGLU>(c, mlp_in, b->wgu, nullptr, nullptr, c->pf_mm, M, 2 * I, H)));
      } else {
        RC(gemm_T<T>(c, mlp_in, b->wgu, nullptr, nullptr, c->pf_gu, M, 2 * I, H));
        RC(launch_pdl(c, swiglu_rows_kernel<T>, dim3(c->sm_count * 4), dim3(256), 0, (const T *)c->pf_gu, (T *)c->pf_mm, (size_t)M * I, f.use_gelu_mlp ? 1 : 0));
      }
      if (b->pfn) {  // olmo2/block.rs:84-86, gemma3/block.rs:130-132: out = x1 + rms_norm(down(...))
        if (use_tc && tc_gemm_ok(M, H, I)) RC((gemm_tc_T<T, TCE_PLAIN>(c, c->pf_mm, b->wd, nullptr, nullptr, c->pf_h, M, H, I)));
        else RC(gemm_T<T>(c, c->pf_mm, b->wd, nullptr, nullptr, c->pf_h, M, H, I));
        RC(launch_pdl(c, rmsnorm_residual_rows_kernel<T>, dim3(M), dim3(256), 0, (const T *)c->pf_h, (const T *)b->pfn, (const T *)c->pf_x1, (T *)x_out, H, f.rms_eps));
      } else if (use_tc && tc_gemm_ok(M, H, I)) RC((gemm_tc_T<T, TCE_RESIDUAL>(c, c->pf_mm, b->wd, nullptr, c->pf_x1, x_out, M, H, I)));
      else RC(gemm_T<T>(c, c->pf_mm, b->wd, nullptr, c->pf_x1, x_out, M, H, I));
      cur = x_out;
    }
    return CAKE_B200_OK;
  });
}


// ------------------------------------------------------------------------------------------ layer-list blocks (fp32 residual stream)
// include/cake_b200.h, cake_b200_layer_spec: parallel block, scalar/vector RMS norm in fp32, token shift, attention with
// soft cap / distance bias / window / keys as values / head gate (attn_window_bias.cuh), gated feed-forward.
static int round_up(int v, int m) { return (v + m - 1) / m * m; }

extern "C" int cake_b200_block_load_spec(cake_b200_ctx *c, int layer_idx, const cake_b200_layer_spec *sp,
                                         const cake_b200_layer_tensors *t, cake_b200_block **out) {
  if (!c || !sp || !t || !out) return fail(CAKE_B200_EINVAL, "null argument");
  if (!c->cfg.layer_list) return fail(CAKE_B200_EINVAL, "block_load_spec needs a ctx created with layer_list = 1");
  if (sp->heads < 1 || sp->kv_heads < 1 || sp->heads % sp->kv_heads || sp->head_dim < 1 || sp->head_dim > WA_MAX_HD)
    return fail(CAKE_B200_EINVAL, "layer %d: heads %d / kv_heads %d / head_dim %d unsupported (heads a multiple of kv_heads, head_dim <= %d)",
                layer_idx, sp->heads, sp->kv_heads, sp->head_dim, WA_MAX_HD);
  if (!sp->values_are_keys || t->v) return fail(CAKE_B200_EINVAL, "layer %d: a separate value projection is not built for layer-list blocks", layer_idx);
  if (sp->window < 0 || sp->ff < 0 || !(sp->scale > 0.f) || sp->softcap < 0.f) return fail(CAKE_B200_EINVAL, "layer %d: bad window / ff / scale / softcap", layer_idx);
  if (!t->norm || !t->q || !t->k || !t->o || (!t->r1) != (!t->r2)) return fail(CAKE_B200_EINVAL, "layer %d: null weight pointer", layer_idx);
  if (sp->ff > 0 && (!t->ff_gate || !t->ff_up || !t->ff_down)) return fail(CAKE_B200_EINVAL, "layer %d: ff = %d but a feed-forward pointer is null", layer_idx, sp->ff);
  CU(cudaSetDevice(c->device));
  const size_t es = c->es, H = c->cfg.hidden, hd = sp->head_dim, sq = (size_t)sp->heads * hd, skv = (size_t)sp->kv_heads * hd, I = sp->ff;
  auto *b = new cake_b200_block{c, layer_idx, c->device};
  b->listed = true;
  b->spec = *sp;
  const int rc = [&]() -> int {
    // one input projection: rows cat(q, k, gate); padded with zero rows to the tensor-core tile so that it can take the shape
    b->n_in = (int)(sq + skv + (t->gate ? sp->heads : 0));
    b->n_in_pad = round_up(b->n_in, b->n_in > 1024 ? 256 : TC_BN);  // wide projections take the 128 x 256 tile
    b->gate_col = t->gate ? (int)(sq + skv) : -1;
    CU(cudaMalloc(&b->w_in, (size_t)b->n_in_pad * H * es + 16));
    CU(cudaMemsetAsync(b->w_in, 0, (size_t)b->n_in_pad * H * es, 0));
    CU(cudaStreamSynchronize(0));
    RC(pipe_copy(c, b->w_in, sq * H * es, t->q, sq * H * es, sq * H * es, 1));
    RC(pipe_copy(c, (char *)b->w_in + sq * H * es, skv * H * es, t->k, skv * H * es, skv * H * es, 1));
    if (t->gate) RC(pipe_copy(c, (char *)b->w_in + (sq + skv) * H * es, sp->heads * H * es, t->gate, sp->heads * H * es, sp->heads * H * es, 1));
    // one output projection over K = heads*hd + ff: row n = [o[n, :], down[n, :]] — mixer and feed-forward of a parallel
    // block add into the same residual, so they are one matrix product over the concatenated activations
    b->k_out = (int)(sq + I);
    CU(cudaMalloc(&b->w_out, H * (sq + I) * es + 16));
    RC(pipe_copy(c, b->w_out, (sq + I) * es, t->o, sq * es, sq * es, H));
    if (I) {
      RC(pipe_copy(c, (char *)b->w_out + sq * es, (sq + I) * es, t->ff_down, I * es, I * es, H));
      CU(cudaMalloc(&b->wgu, 2 * I * H * es + 16));  // row-interleaved gate / up, as cake_b200_block_load lays them out
      RC(pipe_copy(c, b->wgu, 2 * H * es, t->ff_gate, H * es, H * es, I));
      RC(pipe_copy(c, (char *)b->wgu + H * es, 2 * H * es, t->ff_up, H * es, H * es, I));
    }
    RC(upload(c, &b->g, t->norm, (sp->scalar_norm ? 1 : H) * es));
    if (t->shift) RC(upload(c, &b->shift, t->shift, H * es));
    if (t->r1) {
      RC(upload(c, &b->r1, t->r1, sp->heads * es));
      RC(upload(c, &b->r2, t->r2, sp->heads * es));
    }
    return pipe_mark(c);
  }();
  if (rc != CAKE_B200_OK) {
    cake_b200_block_free(b);
    return rc;
  }
  *out = b;
  return CAKE_B200_OK;
}

static int cache_ensure_listed(cake_b200_cache *k, int layer, const cake_b200_block *b) {
  if (layer < 0 || layer >= (int)k->k.size()) return fail(CAKE_B200_EINVAL, "block_idx %d out of range", layer);
  cake_b200_ctx *c = k->ctx;
  const int nkv = b->spec.kv_heads, hd = b->spec.head_dim;
  if (k->k[layer] && (k->kv_heads[layer] != nkv || k->kv_hd[layer] != hd))
    return fail(CAKE_B200_ESTATE, "block_idx %d was used with another layer geometry in this cache", layer);
  if (!k->k[layer]) {
    CU(cudaMalloc(&k->k[layer], (size_t)k->batch * nkv * k->cap * hd * c->es + 16));  // the keys double as values: no V buffer
    k->kv_heads[layer] = nkv;
    k->kv_hd[layer] = hd;
  }
  if (b->shift && !k->shift_state[0][layer])
    for (int i = 0; i < 2; i++) CU(cudaMalloc(&k->shift_state[i][layer], (size_t)k->batch * c->cfg.hidden * sizeof(float)));
  return CAKE_B200_OK;
}

static int sp_reserve(cake_b200_ctx *c, size_t rows, size_t in_cols, size_t out_cols) {
  if (rows <= c->sp_rows && in_cols <= c->sp_in_cols && out_cols <= c->sp_out_cols) return CAKE_B200_OK;
  CU(cudaStreamSynchronize(c->stream));
  rows = std::max(rows, c->sp_rows); in_cols = std::max(in_cols, c->sp_in_cols); out_cols = std::max(out_cols, c->sp_out_cols);
  void **bufs[] = {&c->sp_h, &c->sp_hs, &c->sp_in, &c->sp_a};
  for (void **b : bufs)
    if (*b) { cudaFree(*b); *b = nullptr; }
  c->sp_rows = c->sp_in_cols = c->sp_out_cols = 0;
  const size_t es = c->es, H = c->cfg.hidden;
  CU(cudaMalloc(&c->sp_h, rows * H * es + 16));
  CU(cudaMalloc(&c->sp_hs, rows * H * es + 16));
  CU(cudaMalloc(&c->sp_in, rows * in_cols * es + 16));
  CU(cudaMalloc(&c->sp_a, rows * out_cols * es + 16));
  c->sp_rows = rows; c->sp_in_cols = in_cols; c->sp_out_cols = out_cols;
  return CAKE_B200_OK;
}

// the tcgen05 GEMM takes a product of a layer-list block when D is 16-bit and its tiles cover the shape (N % 128, K % 64);
// CAKE_B200_NO_TC=1 keeps the CUDA-core kernel (A/B aid).  D = float always runs true fp32 on the CUDA cores.
template <typename T> static bool listed_tc(cake_b200_ctx *, int M, int N, int K) {
  static const bool no_tc = []() { const char *e = getenv("CAKE_B200_NO_TC"); return e && e[0] == '1'; }();
  return !no_tc && tc_gemm_ok(M, N, K);
}
template <> bool listed_tc<float>(cake_b200_ctx *, int, int, int) { return false; }
template <typename T, int EPI>
static int listed_gemm_tc(cake_b200_ctx *c, const void *A, const void *W, const void *res, void *C, int M, int N, int K, int act, int ldc,
                          float cap = 0.f, const TcExtra &x = TcExtra{}) {
  return gemm_tc_T<T, EPI>(c, A, W, nullptr, res, C, M, N, K, act, ldc, cap, x);
}
#define NO_TC_F32(EPI) template <> int listed_gemm_tc<float, EPI>(cake_b200_ctx *, const void *, const void *, const void *, void *, int, int, int, int, int, float, const TcExtra &) { return CAKE_B200_EINVAL; }
NO_TC_F32(TCE_PLAIN) NO_TC_F32(TCE_SWIGLU) NO_TC_F32(TCE_RESIDUAL_F32) NO_TC_F32(TCE_SOFTCAP_F32)
#undef NO_TC_F32

// attention of a layer-list block: tensor cores for prompt portions in 16-bit D, the warp-split kernel for steps of a few
// tokens, the warp-per-row kernel for everything else (any head_dim, D = float)
template <typename T> static int listed_attention_mma(cake_b200_ctx *c, const WinAttn &wa, bool *done) {
  *done = true;
  dim3 grid((wa.S + WM_BM - 1) / WM_BM, wa.heads, wa.B), block(WM_THREADS);
  switch (wa.hd) {
    case 32: return launch_pdl(c, attn_window_mma_kernel<T, 32>, grid, block, (size_t)wm_smem_bytes<32>(), wa);
    case 64: return launch_pdl(c, attn_window_mma_kernel<T, 64>, grid, block, (size_t)wm_smem_bytes<64>(), wa);
    case 96: return launch_pdl(c, attn_window_mma_kernel<T, 96>, grid, block, (size_t)wm_smem_bytes<96>(), wa);
    case 128: return launch_pdl(c, attn_window_mma_kernel<T, 128>, grid, block, (size_t)wm_smem_bytes<128>(), wa);
  }
  *done = false;
  return CAKE_B200_OK;
}
template <> int listed_attention_mma<float>(cake_b200_ctx *, const WinAttn &, bool *done) { *done = false; return CAKE_B200_OK; }
// head_dim 128: the tcgen05 kernel (attn_window_tc.cuh); CAKE_B200_FA=mma keeps the mma.sync kernel (A/B aid)
template <typename T> static int listed_attention_tc(cake_b200_ctx *c, const WinAttn &wa, bool *done) {
  static const bool fa_mma = []() { const char *e = getenv("CAKE_B200_FA"); return e && !strcmp(e, "mma"); }();
  static const float fa_tau = []() { const char *e = getenv("CAKE_B200_FA_TAU"); return e ? (float)atof(e) : 5.545f; }();
  *done = false;
  if (fa_mma || wa.hd != FT_HD || wa.ldy % 8 != 0 || wa.kc != wa.vc) return CAKE_B200_OK;
  CUtensorMap mq, mk;
  RC(make_tmap3(&mq, wa.qkg, (uint64_t)wa.ld, (uint64_t)wa.ld, (uint64_t)wa.S, (uint64_t)wa.S, (uint64_t)wa.B, c->cfg.dtype, FT_BM));
  RC(make_tmap3(&mk, wa.kc, (uint64_t)wa.hd, (uint64_t)wa.hd, (uint64_t)(wa.pos0 + wa.S), (uint64_t)wa.cap, (uint64_t)wa.B * wa.n_kv, c->cfg.dtype, FT_BN));
  dim3 gt((wa.S + FT_BM - 1) / FT_BM, wa.heads, wa.B);
  *done = true;
  return launch_pdl(c, attn_window_tc_kernel<T>, gt, dim3(FT_THREADS), (size_t)FT_SMEM_BYTES, mq, mk, mk, wa, fa_tau * 1.4426950408889634f);
}
template <> int listed_attention_tc<float>(cake_b200_ctx *, const WinAttn &, bool *done) { *done = false; return CAKE_B200_OK; }
// attn_window_tc_kernel with its optional parts (kept first keys, sink, a gate buffer, buffers that start at key0).
// kv_row: 0 = kc / vc are caches [B, n_kv, cap, 128]; > 0 = they hold rows of that many elements with the heads side by side
// (one batch row; rows = positions key0 ..).
template <typename T> static int window_attention_tc(cake_b200_ctx *c, const WinAttn &wa, int kv_row, uint64_t *lc) {
  static const float fa_tau = []() { const char *e = getenv("CAKE_B200_FA_TAU"); return e ? (float)atof(e) : 5.545f; }();
  if (wa.hd != FT_HD || wa.ldy % 8 != 0 || wa.ld % 8 != 0 || (kv_row && wa.B != 1) || (wa.gate_mode == 2 && (wa.ldg % 8 != 0 || ((uintptr_t)wa.gate & 15) != 0)))
    return fail(CAKE_B200_EINVAL, "window attention on the tensor cores: shapes not supported");
  CUtensorMap mq, mk, mv;
  const uint64_t vis = (uint64_t)(wa.pos0 + wa.S - wa.key0);
  RC(make_tmap3(&mq, wa.qkg, (uint64_t)wa.ld, (uint64_t)wa.ld, (uint64_t)wa.S, (uint64_t)wa.S, (uint64_t)wa.B, c->cfg.dtype, FT_BM));
  if (kv_row) {
    RC(make_tmap3(&mk, wa.kc, (uint64_t)FT_HD, (uint64_t)kv_row, vis, 0, (uint64_t)wa.n_kv, c->cfg.dtype, FT_BN, (uint64_t)FT_HD));
    RC(make_tmap3(&mv, wa.vc, (uint64_t)FT_HD, (uint64_t)kv_row, vis, 0, (uint64_t)wa.n_kv, c->cfg.dtype, FT_BN, (uint64_t)FT_HD));
  } else {
    RC(make_tmap3(&mk, wa.kc, (uint64_t)FT_HD, (uint64_t)FT_HD, vis, (uint64_t)wa.cap, (uint64_t)wa.B * wa.n_kv, c->cfg.dtype, FT_BN));
    RC(make_tmap3(&mv, wa.vc, (uint64_t)FT_HD, (uint64_t)FT_HD, vis, (uint64_t)wa.cap, (uint64_t)wa.B * wa.n_kv, c->cfg.dtype, FT_BN));
  }
  dim3 gt((wa.S + FT_BM - 1) / FT_BM, wa.heads, wa.B);
  (void)lc;  // launch_pdl counts
  return launch_pdl(c, attn_window_tc_kernel<T>, gt, dim3(FT_THREADS), (size_t)FT_SMEM_BYTES, mq, mk, mv, wa, fa_tau * 1.4426950408889634f);
}
template <> int window_attention_tc<float>(cake_b200_ctx *, const WinAttn &, int, uint64_t *) { return CAKE_B200_EINVAL; }
// steps of a few tokens in 16-bit D with 16-byte rows: eight lanes per key (attn_window_decode_vec_kernel)
template <typename T> static int listed_attention_vec(cake_b200_ctx *c, const WinAttn &wa, bool *done) {
  *done = false;
  if (wa.hd % 8 != 0 || wa.hd > WA_MAX_HD || wa.ld % 8 != 0 || wa.kc != wa.vc || wa.gate_col < -1 ||
      (((uintptr_t)wa.qkg | (uintptr_t)wa.kc) & 15) != 0)
    return CAKE_B200_OK;
  const dim3 grid((unsigned)((long)wa.B * wa.S * wa.heads)), block(WA_DEC_WARPS * 32);
  *done = true;
  switch ((wa.hd + 63) / 64) {
    case 1: return launch_pdl(c, attn_window_decode_vec_kernel<T, 1>, grid, block, 0, wa);
    case 2: return launch_pdl(c, attn_window_decode_vec_kernel<T, 2>, grid, block, 0, wa);
    case 3: return launch_pdl(c, attn_window_decode_vec_kernel<T, 3>, grid, block, 0, wa);
    default: return launch_pdl(c, attn_window_decode_vec_kernel<T, 4>, grid, block, 0, wa);
  }
}
template <> int listed_attention_vec<float>(cake_b200_ctx *, const WinAttn &, bool *done) { *done = false; return CAKE_B200_OK; }
template <typename T> static int listed_attention(cake_b200_ctx *c, const WinAttn &wa) {
  static const bool no_mma = []() { const char *e = getenv("CAKE_B200_NO_TC"); return e && e[0] == '1'; }();
  const long items = (long)wa.B * wa.S * wa.heads;
  if (wa.S >= 16 && !no_mma && wa.ld % 8 == 0 && wa.ldy % 2 == 0) {
    bool done = false;
    RC(listed_attention_tc<T>(c, wa, &done));
    if (done) return CAKE_B200_OK;
    RC(listed_attention_mma<T>(c, wa, &done));
    if (done) return CAKE_B200_OK;
  }
  if (wa.S <= 8 && !no_mma) {
    bool done = false;
    RC(listed_attention_vec<T>(c, wa, &done));
    if (done) return CAKE_B200_OK;
  }
  if (wa.S <= 8) return launch_pdl(c, attn_window_decode_kernel<T>, dim3((unsigned)items), dim3(WA_DEC_WARPS * 32), 0, wa);
  return launch_pdl(c, attn_window_bias_kernel<T>, dim3((unsigned)((items + 3) / 4)), dim3(128), 0, wa);
}

template <typename T, int EPI> static int gemm_rows_T(cake_b200_ctx *c, const RowsGemm &g) {
  dim3 grid((g.N + RG_BN - 1) / RG_BN, (g.M + RG_BM - 1) / RG_BM), block(256);
  return launch_pdl(c, gemm_rows_kernel<T, EPI>, grid, block, 0, g);
}

// x_in, x_out: [B, S, hidden] fp32 (may alias).  Per layer: norm+shift -> input projection -> K append -> attention ->
// gate/up with the activation -> output projection over [attention | feed-forward] with the fp32 residual add.
static int enqueue_listed_layers(cake_b200_ctx *c, cake_b200_block *const *blocks, const int *block_idx, int n,
                                 cake_b200_cache *kc, const float *x_in, float *x_out, int B, int S, int pos0) {
  const int H = c->cfg.hidden, M = B * S;
  size_t in_cols = 0, out_cols = 0;
  for (int i = 0; i < n; i++) {
    in_cols = std::max(in_cols, (size_t)blocks[i]->n_in_pad);
    out_cols = std::max(out_cols, (size_t)blocks[i]->k_out);
  }
  RC(sp_reserve(c, (size_t)M, in_cols, out_cols));
  return DISPATCH_T3(c->cfg.dtype, T_LAMBDA {
    typedef typename decltype(tag_)::type T;
    const float *cur = x_in;
    for (int i = 0; i < n; i++) {
      const cake_b200_block *b = blocks[i];
      const cake_b200_layer_spec &sp = b->spec;
      const int l = block_idx[i], hd = sp.head_dim, sq = sp.heads * hd;
      // 1. h = norm(x) (for the feed-forward) and its token-shifted copy (for the mixer)
      const int cs = kc->shift_cur[l];
      const T *mix_in = (const T *)(b->shift ? c->sp_hs : c->sp_h);
      RC(launch_pdl(c, norm_shift_rows_kernel<T>, dim3(M), dim3(256), 0, cur, (const int *)nullptr, 1, 0, (const T *)b->g, sp.scalar_norm ? 0 : 1,
                    (const T *)b->shift, (const float *)kc->shift_state[cs][l], kc->shift_state[cs ^ 1][l], (T *)c->sp_h, (T *)c->sp_hs, S, H,
                    c->cfg.rms_eps, pos0, 0.f));
      // 2. q | k | gate logits in one product
      RowsGemm gi{mix_in, b->w_in, nullptr, c->sp_in, M, b->n_in, H, H, b->n_in_pad, 0, 0.f};
      if (listed_tc<T>(c, M, b->n_in_pad, H)) RC((listed_gemm_tc<T, TCE_PLAIN>(c, mix_in, b->w_in, nullptr, c->sp_in, M, b->n_in_pad, H, 0, 0)));
      else RC((gemm_rows_T<T, RE_STORE>(c, gi)));
      // 3. the step's keys join the cache, then attention reads keys (= values) only from there
      RC(launch_pdl(c, rows_to_cache_kernel<T>, dim3(M), dim3(128), 0, (const T *)c->sp_in, (T *)kc->k[l], S, b->n_in_pad, sq, sp.kv_heads, hd,
                    kc->cap, pos0));
      WinAttn wa{c->sp_in, kc->k[l], kc->k[l], b->r1, b->r2, c->sp_a, B, S, sp.heads, sp.kv_heads, hd, kc->cap, pos0, b->n_in_pad, b->k_out,
                 b->gate_col, sp.window, sp.scale, sp.softcap};
      RC(listed_attention<T>(c, wa));
      // 4. feed-forward input half: act(gate h) * (up h), written next to the attention output
      if (sp.ff > 0) {
        RowsGemm gu{c->sp_h, b->wgu, nullptr, (T *)c->sp_a + sq, M, 2 * sp.ff, H, H, b->k_out, sp.act, 0.f};
        if (listed_tc<T>(c, M, 2 * sp.ff, H) && sq % 8 == 0 && b->k_out % 8 == 0)
          RC((listed_gemm_tc<T, TCE_SWIGLU>(c, c->sp_h, b->wgu, nullptr, (T *)c->sp_a + sq, M, 2 * sp.ff, H, sp.act, b->k_out)));
        else RC((gemm_rows_T<T, RE_GATE_UP>(c, gu)));
      }
      // 5. x <- x + [attention | ff] . [o | down]^T
      RowsGemm go{c->sp_a, b->w_out, cur, x_out, M, H, b->k_out, b->k_out, H, 0, 0.f};
      if (listed_tc<T>(c, M, H, b->k_out) && (((uintptr_t)cur | (uintptr_t)x_out) & 15) == 0)
        RC((listed_gemm_tc<T, TCE_RESIDUAL_F32>(c, c->sp_a, b->w_out, cur, x_out, M, H, b->k_out, 0, 0)));
      else RC((gemm_rows_T<T, RE_RESIDUAL_F32>(c, go)));
      cur = x_out;
    }
    return CAKE_B200_OK;
  });
}

// ------------------------------------------------------------------------------------------ mixer-list blocks (fp32 residual stream)
// include/cake_b200.h, cake_b200_mixer_spec: sequential pre-norm block; latent attention / retention / state-space mixer
// (kernels in mixers.cu) and a routed feed-forward.  Dense projections run on the GEMMs of the layer-list blocks.
#define MX(call)                                                                                                   \
  do {                                                                                                             \
    int e_ = (call);                                                                                               \
    if (e_ != 0) return fail(CAKE_B200_ECUDA, "%s:%d %s -> %s", __FILE__, __LINE__, #call, cudaGetErrorString((cudaError_t)e_)); \
  } while (0)

// Long portions of a latent-attention layer in 16-bit D run as matrix products on the tensor cores when the tiles cover the
// shapes: scores = qa . cache^T (K = kv_rank + rot_dim), weighted latent = weights . latent (N = kv_rank).
static bool latent_on_tc(const cake_b200_ctx *c, const cake_b200_block *b) {
  static const bool no_tc = []() { const char *e = getenv("CAKE_B200_NO_TC"); return e && e[0] == '1'; }();
  const cake_b200_mixer_spec &sp = b->ms;
  return !no_tc && c->cfg.dtype != CAKE_B200_F32 && sp.kind == CAKE_B200_MIX_LATENT && (sp.kv_rank + sp.rot_dim) % TC_BK == 0 && sp.kv_rank % TC_BN == 0;
}
static int latent_cap_t(int cap) { return (cap + 63) / 64 * 64; }
constexpr int LATENT_TC_ROWS = 4736;     // (token, head) rows per block of the matrix-product form: 37 row tiles x 4 column tiles of the
                                         // weights-times-latent product at rank 512 = one tile per SM
constexpr int LATENT_TC_MIN_ROWS = 1024; // shorter steps take the per-row kernels
constexpr int LATENT_SPLIT_MAX = 32;

// cos / sin of position * frequency for `rows` positions, in double precision, with the optional frequency blend
static void mixer_rope_tables(const cake_b200_rotary_spec &r, int rows, std::vector<float> &cs, std::vector<float> &sn) {
  const int half = r.dims / 2;
  std::vector<double> f(half);
  double amp = 1.0;
  for (int i = 0; i < half; i++) f[i] = pow(r.base, -2.0 * i / r.dims);
  if (r.yarn_factor > 0.0) {
    const double pi = 3.14159265358979323846;
    auto pair_of = [&](double turns) { return r.dims * log((double)r.yarn_original / (2.0 * pi * turns)) / (2.0 * log(r.base)); };
    const double lo = std::max(floor(pair_of(r.yarn_fast)), 0.0), hi = std::min(ceil(pair_of(r.yarn_slow)), (double)(r.dims - 1));
    for (int i = 0; i < half; i++) {
      const double ramp = std::min(1.0, std::max(0.0, (i - lo) / std::max(hi - lo, 0.001)));
      f[i] = f[i] / r.yarn_factor * ramp + f[i] * (1.0 - ramp);
    }
    amp = 0.1 * log(r.yarn_factor) + 1.0;
  }
  cs.resize((size_t)rows * half);
  sn.resize((size_t)rows * half);
  for (int p = 0; p < rows; p++)
    for (int i = 0; i < half; i++) {
      const double a = (double)p * f[i];
      cs[(size_t)p * half + i] = (float)(cos(a) * amp);
      sn[(size_t)p * half + i] = (float)(sin(a) * amp);
    }
}

// the routed feed-forward of a block: norm2, router rows (+ the shared expert's gate row), the stacked experts, the shared expert
static int load_routed_ff(cake_b200_ctx *c, cake_b200_block *b, const cake_b200_moe_spec &mo, const cake_b200_mixer_tensors *t, int layer_idx) {
  const size_t es = c->es, H = c->cfg.hidden;
  const size_t E = mo.experts, Et = E + mo.identity, I = mo.ff, Is = mo.shared_ff;
  RC(upload(c, &b->ln2, t->norm2, H * es));
  // router rows, then the shared expert's gate vector as one more row, zero rows up to the tensor-core tile: one product
  // gives every logit of a token
  const size_t NP = (size_t)round_up((int)Et + 1, TC_BN);
  CU(cudaMalloc(&b->m_router, NP * H * es + 16));
  CU(cudaMemsetAsync(b->m_router, 0, NP * H * es, 0));
  CU(cudaStreamSynchronize(0));
  RC(pipe_copy(c, b->m_router, Et * H * es, t->router, Et * H * es, Et * H * es, 1));
  if (Is) RC(pipe_copy(c, (char *)b->m_router + Et * H * es, H * es, t->s_sg, H * es, H * es, 1));
  RC(upload(c, &b->m_corr, t->correction, Et * es));
  if (E) {
    // all experts stacked: gate / up row-interleaved per expert (as the dense blocks lay theirs out) and the down matrices,
    // so that a grouped product addresses expert e at row e * N of one matrix
    CU(cudaMalloc(&b->m_eg, E * 2 * I * H * es + 16));
    CU(cudaMalloc(&b->m_ed, E * H * I * es + 16));
    for (size_t e = 0; e < E; e++) {
      if (!t->e_gate[e] || !t->e_up[e] || !t->e_down[e]) return fail(CAKE_B200_EINVAL, "layer %d: expert %zu has a null tensor", layer_idx, e);
      char *gu = (char *)b->m_eg + e * 2 * I * H * es;
      RC(pipe_copy(c, gu, 2 * H * es, t->e_gate[e], H * es, H * es, I));
      RC(pipe_copy(c, gu + H * es, 2 * H * es, t->e_up[e], H * es, H * es, I));
      RC(pipe_copy(c, (char *)b->m_ed + e * H * I * es, H * I * es, t->e_down[e], H * I * es, H * I * es, 1));
    }
  }
  if (Is) {  // the shared expert is a dense gated feed-forward: row-interleaved gate / up as everywhere else
    CU(cudaMalloc(&b->wgu, 2 * Is * H * es + 16));
    RC(pipe_copy(c, b->wgu, 2 * H * es, t->s_gate, H * es, H * es, Is));
    RC(pipe_copy(c, (char *)b->wgu + H * es, 2 * H * es, t->s_up, H * es, H * es, Is));
    RC(upload(c, &b->wd, t->s_down, H * Is * es));
  }
  return CAKE_B200_OK;
}

static bool mixer_kind_ext(int kind);
static int load_mixer_ext(cake_b200_ctx *c, int layer_idx, const cake_b200_mixer_spec *sp, const cake_b200_mixer_tensors *t, cake_b200_block **out);
extern "C" int cake_b200_block_load_mixer(cake_b200_ctx *c, int layer_idx, const cake_b200_mixer_spec *sp, const cake_b200_mixer_tensors *t,
                                          cake_b200_block **out) {
  if (!c || !sp || !t || !out) return fail(CAKE_B200_EINVAL, "null argument");
  if (!c->cfg.layer_list) return fail(CAKE_B200_EINVAL, "block_load_mixer needs a ctx created with layer_list = 1");
  if (mixer_kind_ext(sp->kind) || sp->side || sp->norm_offset != 0.f || sp->canon_taps > 0 || sp->dense_ff > 0 || t->post1 || t->post2 ||
      sp->norm_kind != 0 || sp->side_dim > 0)
    return load_mixer_ext(c, layer_idx, sp, t, out);
  const cake_b200_moe_spec &mo = sp->moe;
  const bool has_ff = mo.experts + mo.identity > 0;
  if (sp->heads < 1 || sp->vdim < 1 || !t->norm1 || !t->o) return fail(CAKE_B200_EINVAL, "layer %d: bad heads / vdim or null norm1 / o", layer_idx);
  if (sp->rot.dims < 0 || sp->rot.dims % 2 || (sp->rot.dims > 0 && !(sp->rot.base > 0.0))) return fail(CAKE_B200_EINVAL, "layer %d: bad rotation", layer_idx);
  if (sp->kind == CAKE_B200_MIX_LATENT) {
    if (sp->dim < 1 || sp->rot_dim < 0 || sp->kv_rank < 1 || sp->rot.dims > sp->rot_dim || !t->q || !t->dkv || !t->dkv_norm || !t->uk || !t->uv)
      return fail(CAKE_B200_EINVAL, "layer %d: latent attention needs dim, kv_rank, rot.dims <= rot_dim and q / dkv / dkv_norm / uk / uv", layer_idx);
    if (sp->kv_rank + sp->rot_dim > 768) return fail(CAKE_B200_EINVAL, "layer %d: kv_rank + rot_dim %d > 768", layer_idx, sp->kv_rank + sp->rot_dim);
  } else if (sp->kind == CAKE_B200_MIX_RETENTION) {
    if (sp->dim < 1 || sp->rot.dims > sp->dim || !sp->decay || !t->q || !t->k || !t->v || !t->g)
      return fail(CAKE_B200_EINVAL, "layer %d: retention needs dim, decay, rot.dims <= dim and q / k / v / g", layer_idx);
  } else if (sp->kind == CAKE_B200_MIX_STATE_SPACE) {
    if (sp->state < 1 || sp->groups < 1 || sp->heads % sp->groups || sp->conv < 1 || sp->norm_groups < 1 || (sp->heads * sp->vdim) % sp->norm_groups ||
        !t->in || !t->conv || !t->conv_b || !t->dt_bias || !t->a_log || !t->d || !t->norm)
      return fail(CAKE_B200_EINVAL, "layer %d: state-space mixer needs state, groups | heads, conv, norm_groups | inner and its tensors", layer_idx);
  } else return fail(CAKE_B200_EINVAL, "layer %d: mixer kind %d", layer_idx, sp->kind);
  if (has_ff) {
    if (mo.experts < 0 || mo.identity < 0 || mo.top < 1 || mo.top > mo.experts + mo.identity || mo.top > 32 || mo.experts + mo.identity > 256 ||
        (mo.experts > 0 && mo.ff < 1) || mo.shared_ff < 0 || !t->norm2 || !t->router || !t->correction)
      return fail(CAKE_B200_EINVAL, "layer %d: bad router sizes (top <= 32, experts + identity <= 256) or null norm2 / router / correction", layer_idx);
    if (mo.experts > 0 && (!t->e_gate || !t->e_up || !t->e_down)) return fail(CAKE_B200_EINVAL, "layer %d: null expert table", layer_idx);
    if (mo.shared_ff > 0 && (!t->s_gate || !t->s_up || !t->s_down || !t->s_sg)) return fail(CAKE_B200_EINVAL, "layer %d: null shared-expert pointer", layer_idx);
  }
  CU(cudaSetDevice(c->device));
  const size_t es = c->es, H = c->cfg.hidden;
  auto *b = new cake_b200_block{c, layer_idx, c->device};
  b->mixer = true;
  b->ms = *sp;
  b->ms.decay = nullptr;
  const int rc = [&]() -> int {
    const size_t inner = (size_t)sp->heads * sp->vdim;
    // the fused input projection, zero rows up to the tensor-core tile
    std::vector<std::pair<const void *, size_t>> parts;
    if (sp->kind == CAKE_B200_MIX_LATENT) parts = {{t->q, (size_t)sp->heads * (sp->dim + sp->rot_dim)}, {t->dkv, (size_t)sp->kv_rank + sp->rot_dim}};
    else if (sp->kind == CAKE_B200_MIX_RETENTION) parts = {{t->q, (size_t)sp->heads * sp->dim}, {t->k, (size_t)sp->heads * sp->dim}, {t->v, inner}, {t->g, inner}};
    else parts = {{t->in, 2 * inner + 2 * (size_t)sp->groups * sp->state + sp->heads}};
    size_t n_in = 0;
    for (auto &pr : parts) n_in += pr.second;
    b->n_in = (int)n_in;
    b->n_in_pad = round_up(b->n_in, b->n_in > 1024 ? 256 : TC_BN);
    CU(cudaMalloc(&b->w_in, (size_t)b->n_in_pad * H * es + 16));
    CU(cudaMemsetAsync(b->w_in, 0, (size_t)b->n_in_pad * H * es, 0));
    CU(cudaStreamSynchronize(0));
    size_t row = 0;
    for (auto &pr : parts) {
      RC(pipe_copy(c, (char *)b->w_in + row * H * es, pr.second * H * es, pr.first, pr.second * H * es, pr.second * H * es, 1));
      row += pr.second;
    }
    RC(upload(c, &b->wo, t->o, H * inner * es));
    RC(upload(c, &b->ln1, t->norm1, H * es));
    if (sp->kind == CAKE_B200_MIX_LATENT) {
      RC(upload(c, &b->m_dkv_norm, t->dkv_norm, (size_t)sp->kv_rank * es));
      RC(upload(c, &b->m_uk, t->uk, (size_t)sp->heads * sp->dim * sp->kv_rank * es));
      RC(upload(c, &b->m_uv, t->uv, inner * sp->kv_rank * es));
      if (latent_on_tc(c, b)) {  // the key expansion with kv_rank outermost: the second operand of a plain product per head
        CU(cudaMalloc(&b->m_ukt, (size_t)sp->heads * sp->dim * sp->kv_rank * es + 16));
        RC(pipe_mark(c));
        RC(wait_loads(c));
        MX(mx::transpose_batched(c->stream, c->cfg.dtype, b->m_uk, b->m_ukt, sp->heads, sp->dim, sp->kv_rank, &c->launches));
      }
    } else if (sp->kind == CAKE_B200_MIX_RETENTION) {
      RC(upload(c, (void **)&b->m_decay, sp->decay, sp->heads * sizeof(float)));
    } else {
      const size_t ch = inner + 2 * (size_t)sp->groups * sp->state;
      RC(upload(c, &b->m_conv, t->conv, ch * sp->conv * es));
      RC(upload(c, &b->m_conv_b, t->conv_b, ch * es));
      RC(upload(c, &b->m_dt_bias, t->dt_bias, sp->heads * es));
      RC(upload(c, &b->m_a_log, t->a_log, sp->heads * es));
      RC(upload(c, &b->m_d, t->d, sp->heads * es));
      RC(upload(c, &b->m_norm, t->norm, inner * es));
    }
    if (sp->rot.dims > 0) {
      std::vector<float> cs, sn;
      b->m_rope_rows = c->cfg.max_seq;
      mixer_rope_tables(sp->rot, b->m_rope_rows, cs, sn);
      RC(upload(c, (void **)&b->m_cos, cs.data(), cs.size() * sizeof(float)));
      RC(upload(c, (void **)&b->m_sin, sn.data(), sn.size() * sizeof(float)));
      CU(cudaStreamSynchronize(c->load_stream));  // the staging copy has left the vectors
    }
    if (has_ff) RC(load_routed_ff(c, b, mo, t, layer_idx));
    return pipe_mark(c);
  }();
  if (rc != CAKE_B200_OK) {
    cake_b200_block_free(b);
    return rc;
  }
  *out = b;
  return CAKE_B200_OK;
}

// ------------------------------------------------------------------------------------------ ext blocks
// Mixer-list blocks that use the structure switches of cake_b200_mixer_spec (gains stored as offsets, post norms, the input
// convolution, a side mixer, a dense feed-forward) with the delta / talking-attention / matrix-memory mixers.
static bool mixer_kind_ext(int kind) {
  return kind == CAKE_B200_MIX_DELTA || kind == CAKE_B200_MIX_TALKING_ATTENTION || kind == CAKE_B200_MIX_MATRIX_MEMORY ||
         kind == CAKE_B200_MIX_SINK_ATTENTION || kind == CAKE_B200_MIX_LATENT_WINDOW;
}
static int sub_kv_heads(const cake_b200_mixer_spec &sp) { return sp.kv_heads > 0 ? sp.kv_heads : sp.heads; }

// bucket of a distance: exact below rows / 2, logarithmic from there up to dmax, the last bucket beyond (double precision)
static int distance_bucket(int n, int rows, double dmax) {
  const int half = rows / 2;
  if (n < half) return n;
  if (half < 1 || !(dmax > (double)half)) return rows - 1;
  const double v = floor(log((double)n / half) / log(dmax / half) * (double)(rows - half));
  return (int)std::min<double>(rows - 1, half + v);
}

struct InPart { const void *w; size_t rows; const void *bias; };
// validates one mixer of an ext block, uploads its own tensors into `b` and appends its projections to the fused input product
static int load_sub_mixer(cake_b200_ctx *c, cake_b200_block *b, const cake_b200_mixer_spec *sp, const cake_b200_mixer_tensors *t,
                          std::vector<InPart> &parts, size_t &row, int layer_idx) {
  const size_t es = c->es, H = c->cfg.hidden;
  if (sp->heads < 1 || sp->vdim < 1 || sp->dim < 1 || !t->o) return fail(CAKE_B200_EINVAL, "layer %d: bad heads / dim / vdim or null o", layer_idx);
  const int G = sub_kv_heads(*sp);
  if (G < 1 || sp->heads % G) return fail(CAKE_B200_EINVAL, "layer %d: %d heads over %d key heads", layer_idx, sp->heads, G);
  const size_t inner = (size_t)sp->heads * sp->vdim;
  auto align8 = [&]() {
    const size_t pad = (8 - row % 8) % 8;
    if (pad) { parts.push_back({nullptr, pad, nullptr}); row += pad; }
  };
  auto add = [&](const void *w, size_t rows, const void *bias) -> int {
    const int col = (int)row;
    parts.push_back({w, rows, bias});
    row += rows;
    return col;
  };
  b->ms = *sp;
  b->ms.decay = nullptr;
  b->ms.side = nullptr;
  b->ms.kv_heads = G;
  RC(upload(c, &b->wo, t->o, H * inner * es));
  if (t->branch_norm) RC(upload(c, &b->m_branch, t->branch_norm, H * es));
  if (sp->kind == CAKE_B200_MIX_DELTA) {
    if (sp->conv < 1 || !t->q || !t->k || !t->v || !t->g || !t->q_conv || !t->k_conv || !t->v_conv || !t->beta || !t->a_proj || !t->a_log || !t->dt_bias || !t->norm)
      return fail(CAKE_B200_EINVAL, "layer %d: the delta mixer needs conv >= 1 and q / k / v / g / their convolutions / beta / a_proj / a_log / dt_bias / norm", layer_idx);
    const size_t qk = (size_t)G * sp->dim;
    align8();
    b->pc[0] = add(t->q, qk, nullptr);
    b->pc[1] = add(t->k, qk, nullptr);
    b->pc[2] = add(t->v, inner, nullptr);
    align8();
    b->pc[3] = add(t->g, inner, nullptr);
    align8();
    b->pc[4] = add(t->beta, sp->heads, nullptr);
    align8();
    b->pc[5] = add(t->a_proj, sp->heads, nullptr);
    const size_t ch = 2 * qk + inner, tb = (size_t)sp->conv * es;   // one convolution over the channels q | k | v
    CU(cudaMalloc(&b->m_conv, ch * tb + 16));
    RC(pipe_copy(c, b->m_conv, qk * tb, t->q_conv, qk * tb, qk * tb, 1));
    RC(pipe_copy(c, (char *)b->m_conv + qk * tb, qk * tb, t->k_conv, qk * tb, qk * tb, 1));
    RC(pipe_copy(c, (char *)b->m_conv + 2 * qk * tb, inner * tb, t->v_conv, inner * tb, inner * tb, 1));
    RC(upload(c, &b->m_dt_bias, t->dt_bias, sp->heads * es));
    RC(upload(c, &b->m_a_log, t->a_log, sp->heads * es));
    RC(upload(c, &b->m_norm, t->norm, (size_t)sp->vdim * es));
  } else if (sp->kind == CAKE_B200_MIX_TALKING_ATTENTION) {
    if (!t->q || !t->k || !t->v || (sp->bias_rows > 0 && !t->rel) || sp->bias_rows < 0)
      return fail(CAKE_B200_EINVAL, "layer %d: talking attention needs q / k / v (and rel with bias_rows > 0)", layer_idx);
    align8();
    b->pc[0] = add(t->q, (size_t)sp->heads * sp->dim, t->q_b);
    align8();
    b->pc[1] = add(t->k, (size_t)G * sp->dim, t->k_b);
    align8();
    b->pc[2] = add(t->v, (size_t)G * sp->vdim, t->v_b);
    if (t->g) {
      align8();
      b->pc[3] = add(t->g, inner, nullptr);
    } else b->pc[3] = -1;
    if (t->o_b) RC(upload(c, &b->m_ob, t->o_b, H * es));
    if (t->talk) RC(upload(c, &b->m_talk, t->talk, (size_t)sp->heads * sp->heads * es));
    if (sp->bias_rows > 0) {  // the bias by distance, one row per distance a cached key can have
      const int len = c->cfg.max_seq;
      std::vector<int> bucket(len);
      for (int d = 0; d < len; d++) bucket[d] = distance_bucket(d, sp->bias_rows, (double)sp->bias_max);
      void *rel = nullptr, *bk = nullptr;
      RC(upload(c, &rel, t->rel, (size_t)sp->bias_rows * sp->heads * es));
      int rc = upload(c, &bk, bucket.data(), (size_t)len * sizeof(int));
      if (rc == CAKE_B200_OK) rc = pipe_mark(c);
      if (rc == CAKE_B200_OK) rc = wait_loads(c);
      cudaError_t e = rc == CAKE_B200_OK ? cudaMalloc(&b->m_bias, (size_t)len * sp->heads * sizeof(float)) : cudaSuccess;
      int me = 0;
      if (rc == CAKE_B200_OK && e == cudaSuccess) {
        cudaStreamSynchronize(c->load_stream);  // the staging copy has left `bucket`
        me = mx::distance_bias_table(c->stream, c->cfg.dtype, rel, (const int *)bk, b->m_bias, len, sp->heads, &c->launches);
        cudaStreamSynchronize(c->stream);
      }
      if (rel) cudaFree(rel);
      if (bk) cudaFree(bk);
      if (rc != CAKE_B200_OK) return rc;
      if (e != cudaSuccess || me != 0) return fail(CAKE_B200_ECUDA, "layer %d: distance bias table: %s", layer_idx, cudaGetErrorString(e != cudaSuccess ? e : (cudaError_t)me));
      b->m_bias_len = len;
    }
  } else if (sp->kind == CAKE_B200_MIX_MATRIX_MEMORY) {
    if (!t->q || !t->k || !t->v || !t->g || !t->i_proj || !t->i_b || !t->f_proj || !t->f_b || !t->norm || !(sp->gate_cap > 0.f))
      return fail(CAKE_B200_EINVAL, "layer %d: the matrix memory needs gate_cap > 0 and q / k / v / g / i_proj / i_b / f_proj / f_b / norm", layer_idx);
    if (G != sp->heads) return fail(CAKE_B200_EINVAL, "layer %d: the matrix memory has one key head per head", layer_idx);
    const size_t qk = (size_t)sp->heads * sp->dim;
    align8();
    b->pc[0] = add(t->q, qk, nullptr);
    align8();
    b->pc[1] = add(t->k, qk, nullptr);
    align8();
    b->pc[2] = add(t->v, inner, nullptr);
    align8();
    b->pc[3] = add(t->g, inner, nullptr);
    align8();
    b->pc[4] = add(t->i_proj, sp->heads, nullptr);
    align8();
    b->pc[5] = add(t->f_proj, sp->heads, nullptr);
    RC(upload(c, &b->m_ib, t->i_b, sp->heads * es));
    RC(upload(c, &b->m_fb, t->f_b, sp->heads * es));
    RC(upload(c, &b->m_norm, t->norm, inner * es));
  } else if (sp->kind == CAKE_B200_MIX_SINK_ATTENTION) {
    if (!t->q || !t->k || !t->v || sp->window < 0 || sp->keep_first < 0 || sp->rot.dims < 0 || sp->rot.dims % 2 || sp->rot.dims > sp->dim ||
        (sp->rot.dims > 0 && !(sp->rot.base > 0.0)))
      return fail(CAKE_B200_EINVAL, "layer %d: sink attention needs q / k / v, window and keep_first >= 0 and an even rot.dims <= dim", layer_idx);
    if (std::max(sp->dim, sp->vdim) > 768) return fail(CAKE_B200_EINVAL, "layer %d: head sizes above 768", layer_idx);
    align8();
    b->pc[0] = add(t->q, (size_t)sp->heads * sp->dim, t->q_b);
    align8();
    b->pc[1] = add(t->k, (size_t)G * sp->dim, t->k_b);
    align8();
    b->pc[2] = add(t->v, (size_t)G * sp->vdim, t->v_b);
    if (t->g) {
      align8();
      b->pc[3] = add(t->g, inner, nullptr);
    } else b->pc[3] = -1;
    if (t->sink) RC(upload(c, &b->m_sink, t->sink, (size_t)sp->heads * es));
    if (sp->rot.dims > 0) {
      std::vector<float> cs, sn;
      b->m_rope_rows = c->cfg.max_seq;
      mixer_rope_tables(sp->rot, b->m_rope_rows, cs, sn);
      RC(upload(c, (void **)&b->m_cos, cs.data(), cs.size() * sizeof(float)));
      RC(upload(c, (void **)&b->m_sin, sn.data(), sn.size() * sizeof(float)));
      CU(cudaStreamSynchronize(c->load_stream));  // the staging copy has left the vectors
    }
  } else if (sp->kind == CAKE_B200_MIX_LATENT_WINDOW) {
    if (sp->q_rank < 1 || sp->kv_rank < 1 || sp->kv_rank > 768 || sp->window < 0 || sp->keep_first < 0 || !t->dq || !t->dq_norm || !t->uq || !t->dkv ||
        !t->dkv_norm || !t->uk || !t->uv)
      return fail(CAKE_B200_EINVAL, "layer %d: windowed latent attention needs q_rank, kv_rank <= 768 and dq / dq_norm / uq / dkv / dkv_norm / uk / uv", layer_idx);
    if (G != sp->heads) return fail(CAKE_B200_EINVAL, "layer %d: latent attention expands keys for every head", layer_idx);
    align8();
    b->pc[0] = add(t->dq, (size_t)sp->q_rank, nullptr);
    align8();
    b->pc[1] = add(t->dkv, (size_t)sp->kv_rank, nullptr);
    if (t->g) {
      align8();
      b->pc[3] = add(t->g, (size_t)sp->heads, nullptr);
    } else b->pc[3] = -1;
    RC(upload(c, &b->m_dq_norm, t->dq_norm, (size_t)sp->q_rank * es));
    RC(upload(c, &b->m_uq, t->uq, (size_t)sp->heads * sp->dim * sp->q_rank * es));
    RC(upload(c, &b->m_dkv_norm, t->dkv_norm, (size_t)sp->kv_rank * es));
    RC(upload(c, &b->m_uk, t->uk, (size_t)sp->heads * sp->dim * sp->kv_rank * es));
    RC(upload(c, &b->m_uv, t->uv, inner * sp->kv_rank * es));
  } else return fail(CAKE_B200_EINVAL, "layer %d: mixer kind %d is not built with these block switches", layer_idx, sp->kind);
  return CAKE_B200_OK;
}

static int load_mixer_ext(cake_b200_ctx *c, int layer_idx, const cake_b200_mixer_spec *sp, const cake_b200_mixer_tensors *t, cake_b200_block **out) {
  if (!t->norm1) return fail(CAKE_B200_EINVAL, "layer %d: null norm1", layer_idx);
  const cake_b200_moe_spec &mo = sp->moe;
  const bool has_moe = mo.experts + mo.identity > 0;
  if (has_moe) {
    if (sp->side || sp->canon_taps > 0 || sp->norm_offset != 0.f || sp->dense_ff > 0)
      return fail(CAKE_B200_EINVAL, "layer %d: the routed feed-forward is not built beside a side mixer, an input convolution, offset gains or a dense feed-forward", layer_idx);
    if (mo.experts < 0 || mo.identity < 0 || mo.top < 1 || mo.top > mo.experts + mo.identity || mo.top > 32 || mo.experts + mo.identity > 256 ||
        (mo.experts > 0 && mo.ff < 1) || mo.shared_ff < 0 || mo.act < 0 || mo.act > 2 || !t->norm2 || !t->router || !t->correction)
      return fail(CAKE_B200_EINVAL, "layer %d: bad router sizes (top <= 32, experts + identity <= 256) or null norm2 / router / correction", layer_idx);
    if (mo.experts > 0 && (!t->e_gate || !t->e_up || !t->e_down)) return fail(CAKE_B200_EINVAL, "layer %d: null expert table", layer_idx);
    if (mo.shared_ff > 0 && (!t->s_gate || !t->s_up || !t->s_down || !t->s_sg)) return fail(CAKE_B200_EINVAL, "layer %d: null shared-expert pointer", layer_idx);
  }
  if (sp->norm_kind < 0 || sp->norm_kind > 1) return fail(CAKE_B200_EINVAL, "layer %d: norm_kind %d", layer_idx, sp->norm_kind);
  if (sp->norm_kind == 1) {
    const bool has_ff = has_moe || sp->dense_ff > 0;
    if (sp->side || sp->canon_taps > 0 || sp->norm_offset != 0.f)
      return fail(CAKE_B200_EINVAL, "layer %d: the squashing norm is not built beside a side mixer, an input convolution or offset gains", layer_idx);
    if (!t->norm1_b || (t->post1 && !t->post1_b) || (has_ff && (!t->norm2_b || (t->post2 && !t->post2_b))))
      return fail(CAKE_B200_EINVAL, "layer %d: the squashing norm needs an offset vector beside every gain", layer_idx);
  }
  if (sp->side_dim < 0 || sp->side_col < 0 || (sp->side_dim > 0 && (!t->side_gate || !t->side_proj || !t->side_norm)))
    return fail(CAKE_B200_EINVAL, "layer %d: a token input needs side_gate / side_proj / side_norm", layer_idx);
  if (sp->side && (!t->side || !t->branch_norm || !t->side->branch_norm)) return fail(CAKE_B200_EINVAL, "layer %d: a side mixer needs its tensors and both branch norms", layer_idx);
  if (sp->canon_taps < 0 || (sp->canon_taps > 0 && !t->canon)) return fail(CAKE_B200_EINVAL, "layer %d: canon_taps %d without canon", layer_idx, sp->canon_taps);
  if (sp->dense_ff < 0 || (sp->dense_ff > 0 && (!t->ff_gate || !t->ff_up || !t->ff_down || !t->norm2 || sp->dense_act < 0 || sp->dense_act > 2)))
    return fail(CAKE_B200_EINVAL, "layer %d: a dense feed-forward needs norm2 / ff_gate / ff_up / ff_down and dense_act in 0..2", layer_idx);
  CU(cudaSetDevice(c->device));
  const size_t es = c->es, H = c->cfg.hidden;
  auto *b = new cake_b200_block{c, layer_idx, c->device};
  b->mixer = true;
  b->ext = true;
  const int rc = [&]() -> int {
    std::vector<InPart> parts;
    size_t row = 0;
    RC(load_sub_mixer(c, b, sp, t, parts, row, layer_idx));
    if (sp->side) {
      b->side = new cake_b200_block{c, layer_idx, c->device};
      b->side->mixer = b->side->ext = true;
      RC(load_sub_mixer(c, b->side, sp->side, t->side, parts, row, layer_idx));
    }
    // block-level switches live in the main block's spec
    b->ms.norm_offset = sp->norm_offset;
    b->ms.canon_taps = sp->canon_taps;
    b->ms.dense_ff = sp->dense_ff;
    b->ms.dense_act = sp->dense_act;
    b->ms.dense_limit = sp->dense_limit;
    b->ms.moe = has_moe ? mo : cake_b200_moe_spec{};
    b->ms.norm_kind = sp->norm_kind;
    for (int i = 0; i < 4; i++) b->ms.norm_alpha[i] = sp->norm_alpha[i];
    b->ms.side_dim = sp->side_dim;
    b->ms.side_col = sp->side_col;
    b->n_in = (int)row;
    b->n_in_pad = round_up(b->n_in, b->n_in > 1024 ? 256 : TC_BN);
    CU(cudaMalloc(&b->w_in, (size_t)b->n_in_pad * H * es + 16));
    CU(cudaMemsetAsync(b->w_in, 0, (size_t)b->n_in_pad * H * es, 0));
    bool any_bias = false;
    for (auto &pr : parts) any_bias = any_bias || pr.bias;
    if (any_bias) {
      CU(cudaMalloc(&b->b_in, (size_t)b->n_in_pad * es + 16));
      CU(cudaMemsetAsync(b->b_in, 0, (size_t)b->n_in_pad * es, 0));
    }
    CU(cudaStreamSynchronize(0));
    size_t r = 0;
    for (auto &pr : parts) {
      if (pr.w) RC(pipe_copy(c, (char *)b->w_in + r * H * es, pr.rows * H * es, pr.w, pr.rows * H * es, pr.rows * H * es, 1));
      if (pr.bias) RC(pipe_copy(c, (char *)b->b_in + r * es, pr.rows * es, pr.bias, pr.rows * es, pr.rows * es, 1));
      r += pr.rows;
    }
    RC(upload(c, &b->ln1, t->norm1, H * es));
    if (t->post1) RC(upload(c, &b->post1, t->post1, H * es));
    if (sp->canon_taps > 0) RC(upload(c, &b->canon, t->canon, H * sp->canon_taps * es));
    if (sp->dense_ff > 0) {  // row-interleaved gate / up as everywhere else
      const size_t I = sp->dense_ff;
      RC(upload(c, &b->ln2, t->norm2, H * es));
      if (t->post2) RC(upload(c, &b->post2, t->post2, H * es));
      CU(cudaMalloc(&b->wgu, 2 * I * H * es + 16));
      RC(pipe_copy(c, b->wgu, 2 * H * es, t->ff_gate, H * es, H * es, I));
      RC(pipe_copy(c, (char *)b->wgu + H * es, 2 * H * es, t->ff_up, H * es, H * es, I));
      RC(upload(c, &b->wd, t->ff_down, H * I * es));
    }
    if (has_moe) {
      RC(load_routed_ff(c, b, mo, t, layer_idx));
      if (t->post2) RC(upload(c, &b->post2, t->post2, H * es));
    }
    if (sp->norm_kind == 1) {
      RC(upload(c, &b->ln1_b, t->norm1_b, H * es));
      if (t->post1) RC(upload(c, &b->post1_b, t->post1_b, H * es));
      if (has_moe || sp->dense_ff > 0) {
        RC(upload(c, &b->ln2_b, t->norm2_b, H * es));
        if (t->post2) RC(upload(c, &b->post2_b, t->post2_b, H * es));
      }
    }
    if (sp->side_dim > 0) {
      RC(upload(c, &b->sd_gate, t->side_gate, (size_t)sp->side_dim * H * es));
      RC(upload(c, &b->sd_proj, t->side_proj, H * sp->side_dim * es));
      RC(upload(c, &b->sd_norm, t->side_norm, H * es));
    }
    return pipe_mark(c);
  }();
  if (rc != CAKE_B200_OK) {
    cake_b200_block_free(b);
    return rc;
  }
  *out = b;
  return CAKE_B200_OK;
}

// Long portions of a talking-attention layer in 16-bit D run as matrix products on the tensor cores when the tiles cover the
// shapes: scores = q . keys^T (K = dim), output = weights . values (N = vdim).
static bool talk_on_tc(const cake_b200_ctx *c, const cake_b200_block *b) {
  static const bool no_tc = []() { const char *e = getenv("CAKE_B200_NO_TC"); return e && e[0] == '1'; }();
  const cake_b200_mixer_spec &sp = b->ms;
  return !no_tc && c->cfg.dtype != CAKE_B200_F32 && sp.kind == CAKE_B200_MIX_TALKING_ATTENTION && sp.dim % TC_BK == 0 && sp.vdim % TC_BN == 0;
}
constexpr int TALK_TC_MIN_ROWS = 1024;          // (token, head) rows of a step below which the per-row kernel runs
constexpr size_t TALK_TC_TOKENS = 2048;         // tokens per block: measured best at 4 x 4096 tokens with 8 and with 16 heads (1024: the
                                                // products get small; 4096: more of the causal triangle is wasted)
constexpr size_t TALK_TC_SCORE_BYTES = 1u << 30;  // bound of the fp32 score block: halves the block until it fits

// cache entries of one mixer of an ext block at `slot` (block_idx, or n_layers + block_idx for the side mixer)
static int cache_ensure_sub(cake_b200_cache *k, int slot, const cake_b200_block *b) {
  cake_b200_ctx *c = k->ctx;
  const cake_b200_mixer_spec &sp = b->ms;
  const int G = sp.kv_heads, tag = sp.kind;
  const bool kv_rows = sp.kind == CAKE_B200_MIX_TALKING_ATTENTION || sp.kind == CAKE_B200_MIX_SINK_ATTENTION;
  const int width = kv_rows ? G * (sp.dim + sp.vdim) : sp.kind == CAKE_B200_MIX_LATENT_WINDOW ? sp.kv_rank : sp.heads * sp.dim * sp.vdim;
  if (k->kv_heads[slot] && (k->kv_heads[slot] != tag || k->kv_hd[slot] != width))
    return fail(CAKE_B200_ESTATE, "cache entry %d was used with another layer geometry", slot);
  if (k->kv_heads[slot]) return CAKE_B200_OK;
  if (kv_rows) {
    CU(cudaMalloc(&k->k[slot], (size_t)k->batch * G * k->cap * sp.dim * c->es + 16));
    CU(cudaMalloc(&k->v[slot], (size_t)k->batch * G * k->cap * sp.vdim * c->es + 16));
    if (talk_on_tc(c, b)) CU(cudaMalloc(&k->vt[slot], (size_t)k->batch * G * sp.vdim * latent_cap_t(k->cap) * c->es + 16));
  } else if (sp.kind == CAKE_B200_MIX_LATENT_WINDOW) {  // the normed latent: one row per position for all heads
    CU(cudaMalloc(&k->k[slot], (size_t)k->batch * k->cap * sp.kv_rank * c->es + 16));
  } else {
    CU(cudaMalloc(&k->rec_state[slot], (size_t)k->batch * width * sizeof(float)));
    if (sp.kind == CAKE_B200_MIX_DELTA && sp.conv > 1)
      CU(cudaMalloc(&k->conv_hist[slot], (size_t)k->batch * (sp.conv - 1) * (2 * G * sp.dim + sp.heads * sp.vdim) * c->es + 16));
    if (sp.kind == CAKE_B200_MIX_MATRIX_MEMORY) CU(cudaMalloc(&k->rec_aux[slot], (size_t)k->batch * sp.heads * (sp.dim + 1) * sizeof(float)));
  }
  k->kv_heads[slot] = tag;
  k->kv_hd[slot] = width;
  return CAKE_B200_OK;
}
static int cache_ensure_ext(cake_b200_cache *k, int layer, const cake_b200_block *b) {
  const int nl = (int)k->len.size();
  if ((int)k->k.size() < 2 * nl) return fail(CAKE_B200_EINVAL, "the cache was not created for a layer-list model");
  RC(cache_ensure_sub(k, layer, b));
  if (b->side) RC(cache_ensure_sub(k, nl + layer, b->side));
  if (b->ms.canon_taps > 1 && !k->canon_hist[layer])
    CU(cudaMalloc(&k->canon_hist[layer], (size_t)k->batch * (b->ms.canon_taps - 1) * k->ctx->cfg.hidden * sizeof(float)));
  return CAKE_B200_OK;
}

// scratch of one mixer of an ext block
struct SubScratch {
  void *att, *conv, *qh, *pw, *oh, *cq, *qa, *lat, *kx, *vx;
  float *o32, *qn, *kn, *f1, *f2, *f3, *part, *y, *scores, *stats;
  int nsplit, tc_tok;
};
constexpr int TALK_SPLIT_MAX = 64;
constexpr int WIN_SPLIT_MAX = 32;
// Sink attention and windowed latent attention of a portion on attn_window_tc_kernel: 16-bit D, key and value size 128, a step
// of at least half a query tile; the latent kind expands keys and values of all heads with two products per batch row first.
constexpr int WIN_TC_MIN_ROWS = 64;
static bool window_on_tc(const cake_b200_ctx *c, const cake_b200_block *b, int S) {
  static const bool off = []() {
    const char *e = getenv("CAKE_B200_NO_TC"), *f = getenv("CAKE_B200_FA");
    return (e && e[0] == '1') || (f && !strcmp(f, "mma"));
  }();
  const cake_b200_mixer_spec &sp = b->ms;
  if (off || c->cfg.dtype == CAKE_B200_F32 || S < WIN_TC_MIN_ROWS || sp.dim != FT_HD || sp.vdim != FT_HD || b->n_in_pad % 8 != 0) return false;
  if (sp.kind == CAKE_B200_MIX_SINK_ATTENTION) return b->pc[3] < 0 || b->pc[3] % 8 == 0;
  return sp.kind == CAKE_B200_MIX_LATENT_WINDOW && sp.kv_rank % TC_BK == 0;
}
template <typename Take> static SubScratch sub_scratch(const cake_b200_ctx *c, const cake_b200_block *b, size_t M, int S, int n_keys, Take &&take) {
  SubScratch s{};
  const cake_b200_mixer_spec &sp = b->ms;
  const size_t es = c->es, inner = (size_t)sp.heads * sp.vdim, G = sp.kv_heads;
  s.att = take(M * inner * es);
  s.y = (float *)take(M * c->cfg.hidden * sizeof(float));
  if (sp.kind == CAKE_B200_MIX_SINK_ATTENTION || sp.kind == CAKE_B200_MIX_LATENT_WINDOW) {
    const bool latent = sp.kind == CAKE_B200_MIX_LATENT_WINDOW;
    const size_t vd = latent ? sp.kv_rank : sp.vdim;
    s.qh = take(M * sp.heads * sp.dim * es);  // rotated unit queries / the expanded queries
    if (latent) {
      s.cq = take(M * sp.q_rank * es);
      if (window_on_tc(c, b, S)) {  // keys and values of every head for the rows one batch row's step sees
        const size_t nk = sp.window > 0 ? std::min<size_t>(n_keys, (size_t)S + sp.window - 1) : (size_t)n_keys;
        s.kx = take(nk * sp.heads * sp.dim * es);
        s.vx = take(nk * sp.heads * sp.vdim * es);
      } else {
        s.qa = take(M * sp.heads * sp.kv_rank * es);
        s.lat = take(M * sp.heads * sp.kv_rank * es);
      }
    }
    // steps of a few rows over many visible keys: split the keys so that the step fills the chip
    const int vis = std::min(n_keys, sp.window > 0 ? sp.window + sp.keep_first : n_keys);
    if (M * sp.heads <= 1024 && vis >= 256) {
      s.nsplit = (int)std::min<size_t>(WIN_SPLIT_MAX, std::min<size_t>((vis + 63) / 64, (2 * (size_t)c->sm_count + M * sp.heads - 1) / (M * sp.heads)));
      if (s.nsplit > 1) s.part = (float *)take(M * sp.heads * s.nsplit * (vd + 2) * sizeof(float));
      else s.nsplit = 0;
    }
    return s;
  }
  if (sp.kind == CAKE_B200_MIX_TALKING_ATTENTION) {
    if (talk_on_tc(c, b) && (size_t)S * sp.heads >= TALK_TC_MIN_ROWS) {  // blocks of tc_tok tokens of one batch row as matrix products
      const size_t kp = ((size_t)n_keys + TC_BN - 1) / TC_BN * TC_BN;
      size_t nt = TALK_TC_TOKENS;
      while (nt > TC_BM && sp.heads * nt * kp * sizeof(float) > TALK_TC_SCORE_BYTES) nt /= 2;
      nt = std::min<size_t>((size_t)S, nt);
      s.tc_tok = (int)nt;
      const size_t rows = nt * sp.heads;
      s.qh = take(rows * sp.dim * es);
      s.scores = (float *)take(rows * kp * sizeof(float));
      s.pw = take(rows * 2 * kp * es);
      s.stats = (float *)take(rows * 2 * sizeof(float));
      s.oh = take(rows * sp.vdim * es);
      return s;
    }
    // steps of a few rows over many keys: split the keys so that the step fills the chip
    if (M <= 32 && n_keys >= 256) {
      s.nsplit = (int)std::min<size_t>(TALK_SPLIT_MAX, std::min<size_t>((n_keys + 63) / 64, (2 * (size_t)c->sm_count + M - 1) / M));
      if (s.nsplit > 1) s.part = (float *)take(M * s.nsplit * (2 * (size_t)sp.heads + inner) * sizeof(float));
      else s.nsplit = 0;
    }
    return s;
  }
  s.o32 = (float *)take(M * inner * sizeof(float));
  s.f1 = (float *)take(M * sp.heads * sizeof(float));
  s.f2 = (float *)take(M * sp.heads * sizeof(float));
  if (sp.kind == CAKE_B200_MIX_DELTA) {
    s.conv = take(M * (2 * G * sp.dim + inner) * es);
    s.qn = (float *)take(M * G * sp.dim * sizeof(float));
    s.kn = (float *)take(M * G * sp.dim * sizeof(float));
  } else s.f3 = (float *)take(M * sp.heads * sizeof(float));
  return s;
}
struct MoeScratch {
  void *act, *sact, *sorted;
  float *wts, *sgate, *y, *logits;
  int *ids, *counts, *perm, *pos_of, *tile_expert;
  int max_tiles, tile;
};
static bool moe_on_tc(const cake_b200_ctx *c, const cake_b200_block *b);
template <typename Take> static MoeScratch moe_scratch(const cake_b200_ctx *c, const cake_b200_block *b, size_t M, Take &&take);
template <typename T>
static int enqueue_routed_ff(cake_b200_ctx *c, const cake_b200_block *b, const MoeScratch &w, const void *h, const float *x, float *out, int M, uint64_t *lc);
struct ExtScratch {
  void *h, *proj, *act, *side;
  float *h32;
  SubScratch a, b;
  MoeScratch moe;
  size_t total;
};
static ExtScratch ext_scratch(const cake_b200_ctx *c, const cake_b200_block *b, size_t M, char *base, int S, int n_keys) {
  ExtScratch s{};
  size_t off = 0;
  auto take = [&](size_t bytes) -> void * {
    void *p = base ? base + off : nullptr;
    off += (bytes + 255) / 256 * 256;
    return p;
  };
  const size_t es = c->es, H = c->cfg.hidden;
  s.h = take(M * H * es);
  if (b->ms.canon_taps > 0) s.h32 = (float *)take(M * H * sizeof(float));
  s.proj = take(M * b->n_in_pad * es);
  s.a = sub_scratch(c, b, M, S, n_keys, take);
  if (b->side) s.b = sub_scratch(c, b->side, M, S, n_keys, take);
  if (b->ms.dense_ff > 0) s.act = take(M * (size_t)b->ms.dense_ff * es);
  if (b->ms.side_dim > 0) s.side = take(M * (size_t)b->ms.side_dim * es);
  s.moe = moe_scratch(c, b, M, take);
  s.total = off;
  return s;
}

// C (fp32 [M, N]) = A[M, K] W[N, K]^T
template <typename T> static int gemm_f32_out(cake_b200_ctx *c, const void *A, const void *W, float *C, int M, int N, int K) {
  if (listed_tc<T>(c, M, N, K)) return listed_gemm_tc<T, TCE_SOFTCAP_F32>(c, A, W, nullptr, C, M, N, K, 0, 0);
  RowsGemm g{A, W, nullptr, C, M, N, K, K, N, 0, 0.f};
  return gemm_rows_T<T, RE_SOFTCAP_F32>(c, g);
}
template <typename T> static int gemm_bias_tc(cake_b200_ctx *c, const void *A, const void *W, const void *bias, void *C, int M, int N, int K) {
  return gemm_tc_T<T, TCE_PLAIN>(c, A, W, bias, nullptr, C, M, N, K, 0, 0);
}
template <> int gemm_bias_tc<float>(cake_b200_ctx *, const void *, const void *, const void *, void *, int, int, int) { return CAKE_B200_EINVAL; }

// one mixer of an ext block: proj [M, ldp] holds its projections at b->pc[]; y [M, hidden] fp32 receives o(att) without o's bias
template <typename T>
static int run_sub_mixer(cake_b200_ctx *c, const cake_b200_block *b, cake_b200_cache *kc, int slot, const SubScratch &w, const T *proj, int ldp,
                         int B, int S, int pos0, uint64_t *lc, cudaStream_t st, bool with_out) {
  const cake_b200_mixer_spec &sp = b->ms;
  const int M = B * S, H = c->cfg.hidden, dt = c->cfg.dtype, G = sp.kv_heads, inner = sp.heads * sp.vdim;
  if (sp.kind == CAKE_B200_MIX_DELTA) {
    const int qk = G * sp.dim, ch = 2 * qk + inner;
    const T *cv = (const T *)w.conv;
    mx::ShortConv sc{proj, ldp, b->pc[0], b->m_conv, nullptr, kc->conv_hist[slot], w.conv, B, S, ch, sp.conv, pos0};
    MX(mx::short_conv(st, dt, sc, lc));
    mx::DeltaPrep dp{cv, cv + qk, ch, proj + b->pc[4], proj + b->pc[5], ldp, b->m_a_log, b->m_dt_bias, w.qn, w.kn, w.f1, w.f2, M, sp.heads, G, sp.dim,
                     1.0f / sqrtf((float)sp.dim)};
    MX(mx::delta_prep(st, dt, dp, lc));
    mx::DeltaRule dr{w.qn, w.kn, cv + 2 * qk, ch, w.f1, w.f2, kc->rec_state[slot], w.o32, B, S, sp.heads, G, sp.dim, sp.vdim, pos0};
    MX(mx::delta_rule(st, dt, dr, lc));
    mx::GateNorm gn{w.o32, proj + b->pc[3], ldp, b->m_norm, w.att, M, inner, sp.heads, 0, c->cfg.rms_eps, 0, sp.vdim, nullptr};
    MX(mx::gate_norm(st, dt, gn, lc));
  } else if (sp.kind == CAKE_B200_MIX_TALKING_ATTENTION) {
    RC(launch_pdl(c, rows_to_cache_kernel<T>, dim3(M), dim3(128), 0, proj, (T *)kc->k[slot], S, ldp, b->pc[1], G, sp.dim, kc->cap, pos0));
    RC(launch_pdl(c, rows_to_cache_kernel<T>, dim3(M), dim3(128), 0, proj, (T *)kc->v[slot], S, ldp, b->pc[2], G, sp.vdim, kc->cap, pos0));
    const int cap_t = latent_cap_t(kc->cap);
    if (kc->vt[slot]) MX(mx::values_transposed_append(st, dt, proj, ldp, b->pc[2], kc->vt[slot], B, S, G, sp.vdim, cap_t, pos0, lc));
    if (w.scores && kc->vt[slot]) {
      // blocks of tc_tok tokens: per key head scores = q rows . keys^T on the keys the block's last token sees, softmax + head
      // mixing into w_hi | w_lo, per key head output = [w_hi | w_lo] . values with the values' k coordinate wrapping at kp
      const int grp = sp.heads / G;
      for (int bb = 0; bb < B; bb++)
        for (int t0 = 0; t0 < S; t0 += w.tc_tok) {
          const int n = std::min(w.tc_tok, S - t0), nk = pos0 + t0 + n, kp = round_up(nk, TC_BN);
          const T *pr = proj + ((size_t)bb * S + t0) * ldp;
          MX(mx::rows_by_head(st, dt, pr + b->pc[0], ldp, w.qh, n, sp.heads, sp.dim, lc));
          for (int g = 0; g < G; g++) {
            TcExtra xs;
            xs.w_rows = nk;   // rows past the visible keys read as zeros
            RC((listed_gemm_tc<T, TCE_SOFTCAP_F32>(c, (const T *)w.qh + (size_t)g * grp * n * sp.dim, (const T *)kc->k[slot] + ((size_t)bb * G + g) * kc->cap * sp.dim,
                                                   nullptr, w.scores + (size_t)g * grp * n * kp, grp * n, kp, sp.dim, 0, 0, 0.f, xs)));
          }
          mx::TalkSoftmax sm{w.scores, w.pw, w.stats, b->m_bias, b->m_bias_len, b->m_talk, n, sp.heads, kp, pos0 + t0, sp.scale};
          MX(mx::talk_softmax(st, dt, sm, lc));
          for (int g = 0; g < G; g++) {
            TcExtra xv;
            xv.b_kwrap = kp;
            xv.w_cols = nk;
            xv.w_ld = cap_t;
            RC((listed_gemm_tc<T, TCE_PLAIN>(c, (const T *)w.pw + (size_t)g * grp * n * 2 * kp, (const T *)kc->vt[slot] + ((size_t)bb * G + g) * sp.vdim * cap_t, nullptr,
                                             (T *)w.oh + (size_t)g * grp * n * sp.vdim, grp * n, sp.vdim, 2 * kp, 0, 0, 0.f, xv)));
          }
          MX(mx::rows_to_tokens(st, dt, w.oh, b->pc[3] >= 0 ? pr + b->pc[3] : nullptr, ldp, (T *)w.att + ((size_t)bb * S + t0) * inner, inner, n, sp.heads, sp.vdim, lc));
        }
    } else {
      mx::TalkAttn ta{proj + b->pc[0], ldp, kc->k[slot], kc->v[slot], b->pc[3] >= 0 ? proj + b->pc[3] : nullptr, ldp, b->m_bias, b->m_bias_len, b->m_talk,
                      w.att, B, S, sp.heads, G, sp.dim, sp.vdim, kc->cap, pos0, sp.scale, w.part, w.nsplit};
      MX(mx::talk_attention(st, dt, ta, lc));
    }
  } else if (sp.kind == CAKE_B200_MIX_SINK_ATTENTION) {
    mx::QkPrep qp{proj, ldp, b->pc[0], b->pc[1], b->pc[2], b->m_cos, b->m_sin, sp.rot.dims, sp.qk_unit, c->cfg.rms_eps, w.qh, kc->k[slot], kc->v[slot],
                  B, S, sp.heads, G, sp.dim, sp.vdim, kc->cap, pos0};
    MX(mx::qk_prep(st, dt, qp, lc));
    mx::WindowAttn wa{w.qh, sp.heads * sp.dim, kc->k[slot], kc->v[slot], b->pc[3] >= 0 ? proj + b->pc[3] : nullptr, ldp, 0, b->m_sink, w.att, inner,
                      B, S, sp.heads, G, sp.dim, sp.vdim, kc->cap, pos0, sp.window, sp.keep_first, sp.scale, w.part, w.nsplit};
    if (window_on_tc(c, b, S)) {
      const void *gate = b->pc[3] >= 0 ? proj + b->pc[3] : nullptr;
      WinAttn ta{w.qh, kc->k[slot], kc->v[slot], nullptr, nullptr, w.att, B, S, sp.heads, G, FT_HD, kc->cap, pos0, sp.heads * FT_HD, inner, -1, sp.window,
                 sp.scale, 0.f, sp.keep_first, 0, b->m_sink, gate, gate ? 2 : 0, ldp};
      RC(window_attention_tc<T>(c, ta, 0, lc));
    } else if (mx::window_attention_tiled_ok(dt, wa)) MX(mx::window_attention_tiled(st, dt, wa, lc));
    else MX(mx::window_attention(st, dt, wa, lc));
  } else if (sp.kind == CAKE_B200_MIX_LATENT_WINDOW) {
    // both latents are normed (the key / value latent straight into the cache), the query latent is expanded and taken through
    // the key expansion, so that the attention runs over the cached latent rows for all heads: qa_h = uk_h^T q_h,
    // lat_h = sum_j w_hj c_j, att_h = uv_h lat_h
    const int R = sp.kv_rank;
    mx::RmsCols nq{proj, ldp, b->pc[0], b->m_dq_norm, w.cq, sp.q_rank, S, 0, M, S, sp.q_rank, c->cfg.rms_eps};
    MX(mx::rms_cols(st, dt, nq, lc));
    mx::RmsCols nk{proj, ldp, b->pc[1], b->m_dkv_norm, kc->k[slot], R, kc->cap, pos0, M, S, R, c->cfg.rms_eps};
    MX(mx::rms_cols(st, dt, nk, lc));
    if (listed_tc<T>(c, M, sp.heads * sp.dim, sp.q_rank)) RC((listed_gemm_tc<T, TCE_PLAIN>(c, w.cq, b->m_uq, nullptr, w.qh, M, sp.heads * sp.dim, sp.q_rank, 0, 0)));
    else {
      RowsGemm gq{w.cq, b->m_uq, nullptr, w.qh, M, sp.heads * sp.dim, sp.q_rank, sp.q_rank, sp.heads * sp.dim, 0, 0.f};
      RC((gemm_rows_T<T, RE_STORE>(c, gq)));
    }
    if (window_on_tc(c, b, S)) {
      // a portion: k = uk c and v = uv c of all heads for the rows the step sees (two products per batch row), then the
      // windowed attention over them with a gate per head
      const int key0 = sp.window > 0 ? std::max(0, pos0 - sp.window + 1) : 0, nk = pos0 + S - key0, qw = sp.heads * FT_HD;
      for (int bb = 0; bb < B; bb++) {
        const T *rows = (const T *)kc->k[slot] + ((size_t)bb * kc->cap + key0) * R;
        RC((listed_gemm_tc<T, TCE_PLAIN>(c, rows, b->m_uk, nullptr, w.kx, nk, qw, R, 0, 0)));
        RC((listed_gemm_tc<T, TCE_PLAIN>(c, rows, b->m_uv, nullptr, w.vx, nk, qw, R, 0, 0)));
        const void *gate = b->pc[3] >= 0 ? proj + (size_t)bb * S * ldp + b->pc[3] : nullptr;
        WinAttn ta{(const T *)w.qh + (size_t)bb * S * qw, w.kx, w.vx, nullptr, nullptr, (T *)w.att + (size_t)bb * S * inner, 1, S, sp.heads, sp.heads, FT_HD, nk,
                   pos0, qw, inner, -1, sp.window, sp.scale, 0.f, 0, key0, nullptr, gate, gate ? 1 : 0, ldp};
        RC(window_attention_tc<T>(c, ta, qw, lc));
      }
      return with_out ? gemm_f32_out<T>(c, w.att, b->wo, w.y, M, H, inner) : CAKE_B200_OK;
    }
    mx::HeadGemm ga{w.qh, b->m_uk, w.qa, M, R, sp.dim, sp.heads, sp.dim, (long)sp.dim * R, R, sp.heads * sp.dim, R, sp.heads * R, 1};
    MX(mx::head_gemm(st, dt, ga, lc));
    mx::WindowAttn wa{w.qa, sp.heads * R, kc->k[slot], kc->k[slot], b->pc[3] >= 0 ? proj + b->pc[3] : nullptr, ldp, 1, nullptr, w.lat, sp.heads * R,
                      B, S, sp.heads, 1, R, R, kc->cap, pos0, sp.window, sp.keep_first, sp.scale, w.part, w.nsplit};
    if (mx::window_attention_tiled_ok(dt, wa)) MX(mx::window_attention_tiled(st, dt, wa, lc));
    else MX(mx::window_attention(st, dt, wa, lc));
    mx::HeadGemm gv{w.lat, b->m_uv, w.att, M, sp.vdim, R, sp.heads, R, (long)sp.vdim * R, sp.vdim, sp.heads * R, R, inner, 0};
    MX(mx::head_gemm(st, dt, gv, lc));
  } else {
    const float qs = 1.0f / sqrtf((float)sp.dim);
    mx::GatePrep gp{proj + b->pc[0], proj + b->pc[1], ldp, proj + b->pc[4], proj + b->pc[5], ldp, b->m_ib, b->m_fb, kc->rec_aux[slot], w.f1, w.f2, w.f3,
                    B, S, sp.heads, sp.dim, pos0, sp.gate_cap, qs};
    MX(mx::gate_prep(st, dt, gp, lc));
    mx::Recurrence r{proj + b->pc[0], proj + b->pc[1], proj + b->pc[2], ldp, ldp, ldp, 1, nullptr, 0, nullptr, nullptr, nullptr, nullptr, 1.0f,
                     nullptr, nullptr, 0, kc->rec_state[slot], w.o32, B, S, sp.heads, sp.dim, sp.vdim, pos0, w.f1, w.f2};
    MX(mx::recurrence(st, dt, r, lc));
    mx::GateNorm gn{w.o32, proj + b->pc[3], ldp, b->m_norm, w.att, M, inner, sp.heads, 0, c->cfg.rms_eps, 1, 0, w.f3};
    MX(mx::gate_norm(st, dt, gn, lc));
  }
  return with_out ? gemm_f32_out<T>(c, w.att, b->wo, w.y, M, H, inner) : CAKE_B200_OK;
}

// one ext block: x_out = x + post1(mixers(canon(norm1(x)))), then x_out += post2(ff(norm2(x_out)))
template <typename T>
static int enqueue_ext_layer(cake_b200_ctx *c, const cake_b200_block *b, int l, cake_b200_cache *kc, const float *cur, float *x_out, int B, int S, int pos0,
                             uint64_t *lc) {
  const cake_b200_mixer_spec &sp = b->ms;
  const int M = B * S, H = c->cfg.hidden, dt = c->cfg.dtype, nl = (int)kc->len.size();
  const float eps = c->cfg.rms_eps;
  cudaStream_t st = c->stream;
  const ExtScratch w = ext_scratch(c, b, (size_t)M, (char *)c->mx_ws, S, pos0 + S);
  // 1. h = norm1(x), the input convolution, every projection of the mixer(s) in one product
  const bool squash = sp.norm_kind == 1;  // tanh(alpha x) * w + b instead of an RMS norm, in all four places
  if (squash) {
    mx::TanhNorm n1{cur, nullptr, 1, 0, b->ln1, b->ln1_b, sp.norm_alpha[0], nullptr, nullptr, w.h, M, H};
    MX(mx::tanh_norm(st, dt, n1, lc));
  } else {
    mx::RmsRows n1{cur, b->ln1, sp.norm_offset, sp.canon_taps > 0 ? w.h32 : nullptr, sp.canon_taps > 0 ? nullptr : w.h, M, H, eps};
    MX(mx::rms_rows(st, dt, n1, lc));
  }
  if (sp.canon_taps > 0) {
    mx::CanonConv cc{w.h32, b->canon, kc->canon_hist[l], w.h, B, S, H, sp.canon_taps, pos0};
    MX(mx::canon_conv(st, dt, cc, lc));
  }
  if (listed_tc<T>(c, M, b->n_in_pad, H)) RC(gemm_bias_tc<T>(c, w.h, b->w_in, b->b_in, w.proj, M, b->n_in_pad, H));
  else {
    RowsGemm gi{w.h, b->w_in, nullptr, w.proj, M, b->n_in, H, H, b->n_in_pad, 0, 0.f, nullptr, b->b_in};
    RC((gemm_rows_T<T, RE_STORE>(c, gi)));
  }
  // 2. the mixer(s), each up to its output projection in fp32
  // a recurrent side mixer (its kernels take a stream; its few CTAs leave most of the chip idle) runs next to the main mixer
  const bool fork = b->side && b->side->ms.kind != CAKE_B200_MIX_TALKING_ATTENTION && M >= 256 && !c->capturing;
  if (fork) {
    if (!c->side_stream) {
      CU(cudaStreamCreateWithFlags(&c->side_stream, cudaStreamNonBlocking));
      CU(cudaEventCreateWithFlags(&c->ev_fork, cudaEventDisableTiming));
      CU(cudaEventCreateWithFlags(&c->ev_join, cudaEventDisableTiming));
    }
    CU(cudaEventRecord(c->ev_fork, st));
    CU(cudaStreamWaitEvent(c->side_stream, c->ev_fork, 0));
    RC(run_sub_mixer<T>(c, b->side, kc, nl + l, w.b, (const T *)w.proj, b->n_in_pad, B, S, pos0, lc, c->side_stream, false));
    CU(cudaEventRecord(c->ev_join, c->side_stream));
  }
  RC(run_sub_mixer<T>(c, b, kc, l, w.a, (const T *)w.proj, b->n_in_pad, B, S, pos0, lc, st, true));
  if (fork) {
    CU(cudaStreamWaitEvent(st, c->ev_join, 0));
    RC(gemm_f32_out<T>(c, w.b.att, b->side->wo, w.b.y, M, H, b->side->ms.heads * b->side->ms.vdim));
  } else if (b->side) RC(run_sub_mixer<T>(c, b->side, kc, nl + l, w.b, (const T *)w.proj, b->n_in_pad, B, S, pos0, lc, st, true));
  // 3. x <- x + post1(branches)
  if (squash && b->post1) {
    mx::TanhNorm p1{w.a.y, nullptr, 1, 0, b->post1, b->post1_b, sp.norm_alpha[1], cur, x_out, nullptr, M, H};
    MX(mx::tanh_norm(st, dt, p1, lc));
  } else {
    mx::BranchMerge bm{w.a.y, b->side ? w.b.y : nullptr, b->m_ob, b->side ? b->side->m_ob : nullptr, b->m_branch, b->side ? b->side->m_branch : nullptr,
                       b->post1, sp.norm_offset, cur, x_out, M, H, eps};
    MX(mx::branch_merge(st, dt, bm, lc));
  }
  // 4. x <- x + post2(ff(norm2(x)))
  const bool has_moe = sp.moe.experts + sp.moe.identity > 0;
  if (sp.dense_ff > 0 || has_moe) {
    if (squash) {
      mx::TanhNorm n2{x_out, nullptr, 1, 0, b->ln2, b->ln2_b, sp.norm_alpha[2], nullptr, nullptr, w.h, M, H};
      MX(mx::tanh_norm(st, dt, n2, lc));
    } else {
      mx::RmsRows n2{x_out, b->ln2, sp.norm_offset, nullptr, w.h, M, H, eps};
      MX(mx::rms_rows(st, dt, n2, lc));
    }
  }
  if (has_moe) {  // the feed-forward's sum lands in y; a post norm squashes it on its way into the stream
    if (b->post2) {
      RC(enqueue_routed_ff<T>(c, b, w.moe, w.h, nullptr, w.a.y, M, lc));
      if (squash) {
        mx::TanhNorm p2{w.a.y, nullptr, 1, 0, b->post2, b->post2_b, sp.norm_alpha[3], x_out, x_out, nullptr, M, H};
        MX(mx::tanh_norm(st, dt, p2, lc));
      } else {
        mx::BranchMerge fm{w.a.y, nullptr, nullptr, nullptr, nullptr, nullptr, b->post2, sp.norm_offset, x_out, x_out, M, H, eps};
        MX(mx::branch_merge(st, dt, fm, lc));
      }
    } else RC(enqueue_routed_ff<T>(c, b, w.moe, w.h, x_out, x_out, M, lc));
  }
  if (sp.dense_ff > 0) {
    const int I = sp.dense_ff;
    if (listed_tc<T>(c, M, 2 * I, H)) RC((listed_gemm_tc<T, TCE_SWIGLU>(c, w.h, b->wgu, nullptr, w.act, M, 2 * I, H, sp.dense_act, I, sp.dense_limit)));
    else {
      RowsGemm gu{w.h, b->wgu, nullptr, w.act, M, 2 * I, H, H, I, sp.dense_act, sp.dense_limit};
      RC((gemm_rows_T<T, RE_GATE_UP>(c, gu)));
    }
    RC(gemm_f32_out<T>(c, w.act, b->wd, w.a.y, M, H, I));
    if (squash && b->post2) {
      mx::TanhNorm p2{w.a.y, nullptr, 1, 0, b->post2, b->post2_b, sp.norm_alpha[3], x_out, x_out, nullptr, M, H};
      MX(mx::tanh_norm(st, dt, p2, lc));
    } else {
      mx::BranchMerge fm{w.a.y, nullptr, nullptr, nullptr, nullptr, nullptr, b->post2, sp.norm_offset, x_out, x_out, M, H, eps};
      MX(mx::branch_merge(st, dt, fm, lc));
    }
  }
  // 5. the per-layer token input
  if (sp.side_dim > 0) {
    if (!c->side_tab || sp.side_col + sp.side_dim > c->side_cols) return fail(CAKE_B200_ESTATE, "layer %d: the token input needs columns %d..%d of the side table (%d loaded)", b->layer, sp.side_col, sp.side_col + sp.side_dim, c->side_cols);
    if (c->d_ids_n != (size_t)M) return fail(CAKE_B200_ESTATE, "layer %d: the token input needs the ids of this step (%zu embedded, %d rows)", b->layer, c->d_ids_n, M);
    // g = gelu(G x) * e and y = P g as two products with the gate between them; x += rms(y) * w is a merge with a post norm
    const int sd = sp.side_dim;
    const void *xa = x_out;  // D = float: the stream is the operand as it stands
    if (dt != CAKE_B200_F32) {
      MX(mx::rows_to_d(st, dt, x_out, w.h, (size_t)M * H, lc));
      xa = w.h;
    }
    if (listed_tc<T>(c, M, sd, H)) RC((listed_gemm_tc<T, TCE_PLAIN>(c, xa, b->sd_gate, nullptr, w.side, M, sd, H, 0, 0)));
    else {
      RowsGemm gg{xa, b->sd_gate, nullptr, w.side, M, sd, H, H, sd, 0, 0.f};
      RC((gemm_rows_T<T, RE_STORE>(c, gg)));
    }
    mx::SideGate sg{w.side, sd, c->d_ids, c->side_tab, c->side_cols, sp.side_col, M, sd};
    MX(mx::side_gate(st, dt, sg, lc));
    RC(gemm_f32_out<T>(c, w.side, b->sd_proj, w.a.y, M, H, sd));
    mx::BranchMerge sm{w.a.y, nullptr, nullptr, nullptr, nullptr, nullptr, b->sd_norm, 0.f, x_out, x_out, M, H, eps};
    MX(mx::branch_merge(st, dt, sm, lc));
  }
  return CAKE_B200_OK;
}

static int cache_ensure_mixer(cake_b200_cache *k, int layer, const cake_b200_block *b) {
  if (layer < 0 || layer >= (int)k->len.size()) return fail(CAKE_B200_EINVAL, "block_idx %d out of range", layer);
  if (b->ext) return cache_ensure_ext(k, layer, b);
  cake_b200_ctx *c = k->ctx;
  const cake_b200_mixer_spec &sp = b->ms;
  // (kind, row width) a slot was first used with: a slot never changes its layer
  const int tag = sp.kind, width = sp.kind == CAKE_B200_MIX_LATENT ? sp.kv_rank + sp.rot_dim
                                  : sp.heads * (sp.kind == CAKE_B200_MIX_RETENTION ? sp.dim : sp.state) * sp.vdim;
  if (k->kv_heads[layer] && (k->kv_heads[layer] != tag || k->kv_hd[layer] != width))
    return fail(CAKE_B200_ESTATE, "block_idx %d was used with another layer geometry in this cache", layer);
  if (k->kv_heads[layer]) return CAKE_B200_OK;
  if (sp.kind == CAKE_B200_MIX_LATENT) {
    CU(cudaMalloc(&k->k[layer], (size_t)k->batch * k->cap * width * c->es + 16));
    // the latent once more with the positions innermost, for the matrix-product form of long portions (latent_on_tc)
    if (latent_on_tc(c, b)) CU(cudaMalloc(&k->v[layer], (size_t)k->batch * sp.kv_rank * latent_cap_t(k->cap) * c->es + 16));
  } else {
    CU(cudaMalloc(&k->rec_state[layer], (size_t)k->batch * width * sizeof(float)));
    if (sp.kind == CAKE_B200_MIX_STATE_SPACE && sp.conv > 1)
      CU(cudaMalloc(&k->conv_hist[layer], (size_t)k->batch * (sp.conv - 1) * (sp.heads * sp.vdim + 2 * sp.groups * sp.state) * c->es + 16));
  }
  k->kv_heads[layer] = tag;
  k->kv_hd[layer] = width;
  return CAKE_B200_OK;
}

// scratch of one block for M rows, carved from the ctx arena (base == nullptr: sizes only)
struct MixerScratch {
  void *h, *proj, *qa, *lat, *att, *conv, *pw;
  float *o32, *part, *scores;
  int nsplit, lat_tok;
  MoeScratch moe;
  size_t total;
};
// the routed experts of a block run as grouped products on the tensor cores when D is 16-bit and the tiles cover the shapes
static bool moe_on_tc(const cake_b200_ctx *c, const cake_b200_block *b) {
  static const bool no_tc = []() { const char *e = getenv("CAKE_B200_NO_TC"); return e && e[0] == '1'; }();
  const cake_b200_moe_spec &mo = b->ms.moe;
  return !no_tc && c->cfg.dtype != CAKE_B200_F32 && mo.experts > 0 && c->cfg.hidden % 128 == 0 && mo.ff % 64 == 0;
}
template <typename Take> static MoeScratch moe_scratch(const cake_b200_ctx *c, const cake_b200_block *b, size_t M, Take &&take) {
  MoeScratch s{};
  const cake_b200_moe_spec &mo = b->ms.moe;
  if (mo.experts + mo.identity < 1) return s;
  const size_t es = c->es, H = c->cfg.hidden, nt = M * mo.top;
  s.tile = moe_on_tc(c, b) ? TC_BM : 64;
  s.max_tiles = (int)((nt + s.tile - 1) / s.tile + std::min<size_t>(mo.experts, nt));
  const size_t rows = (size_t)s.max_tiles * s.tile;
  s.logits = (float *)take(M * (size_t)round_up(mo.experts + mo.identity + 1, TC_BN) * sizeof(float));
  s.ids = (int *)take(nt * sizeof(int));
  s.wts = (float *)take(nt * sizeof(float));
  s.sgate = (float *)take(M * sizeof(float));
  s.counts = (int *)take((mo.experts + 1) * sizeof(int));
  s.perm = (int *)take(rows * sizeof(int));
  s.pos_of = (int *)take(nt * sizeof(int));
  s.tile_expert = (int *)take(s.max_tiles * sizeof(int));
  if (mo.experts) {
    s.act = take(rows * mo.ff * es);
    s.y = (float *)take(rows * H * sizeof(float));
    if (s.tile == TC_BM) s.sorted = take(rows * H * es);
  }
  if (mo.shared_ff) s.sact = take(M * mo.shared_ff * es);
  return s;
}
static MixerScratch mixer_scratch(const cake_b200_ctx *c, const cake_b200_block *b, size_t M, char *base, int S = 1, int n_keys = 1) {
  MixerScratch s{};
  size_t off = 0;
  auto take = [&](size_t bytes) -> void * {
    void *p = base ? base + off : nullptr;
    off += (bytes + 255) / 256 * 256;
    return p;
  };
  const cake_b200_mixer_spec &sp = b->ms;
  const size_t es = c->es, H = c->cfg.hidden, inner = (size_t)sp.heads * sp.vdim;
  s.h = take(M * H * es);
  s.proj = take(M * b->n_in_pad * es);
  s.att = take(M * inner * es);
  if (sp.kind == CAKE_B200_MIX_LATENT) {
    s.qa = take(M * sp.heads * (sp.kv_rank + sp.rot_dim) * es);
    s.lat = take(M * sp.heads * sp.kv_rank * es);
    if (latent_on_tc(c, b) && (size_t)S * sp.heads >= LATENT_TC_MIN_ROWS) {
      s.lat_tok = std::max(1, std::min(S, LATENT_TC_ROWS / sp.heads));
      const size_t rows = (size_t)s.lat_tok * sp.heads, kp = ((size_t)n_keys + TC_BN - 1) / TC_BN * TC_BN;
      s.scores = (float *)take(rows * kp * sizeof(float));
      s.pw = take(rows * 2 * kp * es);
    } else if (M * sp.heads <= 2048 && n_keys > 128) {
      s.nsplit = std::min(LATENT_SPLIT_MAX, (n_keys + 127) / 128);
      s.part = (float *)take(M * sp.heads * s.nsplit * (sp.kv_rank + 2) * sizeof(float));
    }
  } else {
    s.o32 = (float *)take(M * inner * sizeof(float));
    if (sp.kind == CAKE_B200_MIX_STATE_SPACE) s.conv = take(M * (inner + 2 * (size_t)sp.groups * sp.state) * es);
  }
  s.moe = moe_scratch(c, b, M, take);
  s.total = off;
  return s;
}

// The routed feed-forward on normed rows h [M, hidden] in D: out = (x ? x : 0) + sum over a token's chosen experts of weight *
// expert(h) (+ weight * h for identity experts) + sigmoid(shared gate) * shared expert(h); out may alias x.
template <typename T>
static int enqueue_routed_ff(cake_b200_ctx *c, const cake_b200_block *b, const MoeScratch &w, const void *h, const float *x, float *out, int M, uint64_t *lc) {
  const cake_b200_moe_spec &mo = b->ms.moe;
  const int H = c->cfg.hidden, dt = c->cfg.dtype;
  cudaStream_t st = c->stream;
  const int NP = round_up(mo.experts + mo.identity + 1, TC_BN);
  RowsGemm gr{h, b->m_router, nullptr, w.logits, M, NP, H, H, NP, 0, 0.f};
  if (listed_tc<T>(c, M, NP, H)) RC((listed_gemm_tc<T, TCE_SOFTCAP_F32>(c, h, b->m_router, nullptr, w.logits, M, NP, H, 0, 0)));
  else RC((gemm_rows_T<T, RE_SOFTCAP_F32>(c, gr)));
  mx::MoePlan mp{w.logits, NP, b->m_corr, mo.shared_ff ? 1 : 0, M, H, mo.experts, mo.identity, mo.top, mo.scale, w.ids, w.wts,
                 w.sgate, w.tile, w.counts, w.perm, w.pos_of, w.tile_expert, w.max_tiles, mo.logit_bias};
  MX(mx::moe_route(st, dt, mp, lc));
  if (mo.experts && w.sorted) {  // grouped products: sorted rows of h -> act(gate) * up -> down, expert e at row e * N of the stacked weights
    const int rows = w.max_tiles * w.tile;
    MX(mx::moe_gather(st, dt, h, w.perm, w.sorted, rows, H, mo.top, lc));
    TcExtra xg;
    xg.tile_group = w.tile_expert;
    xg.n_groups = mo.experts;
    RC((listed_gemm_tc<T, TCE_SWIGLU>(c, w.sorted, b->m_eg, nullptr, w.act, rows, 2 * mo.ff, H, mo.act, mo.ff, mo.limit, xg)));
    RC((listed_gemm_tc<T, TCE_SOFTCAP_F32>(c, w.act, b->m_ed, nullptr, w.y, rows, H, mo.ff, 0, 0, 0.f, xg)));
  } else if (mo.experts) {
    mx::MoeExperts me{h, b->m_eg, b->m_ed, w.act, w.y, M, H, mo.ff, mo.top, mo.act, w.perm, w.tile_expert, w.tile, w.max_tiles, mo.limit};
    MX(mx::moe_experts(st, dt, me, lc));
  }
  mx::MoeCombine mc{x, out, h, w.y, w.wts, w.ids, w.pos_of, M, H, mo.top, mo.experts};
  MX(mx::moe_combine(st, dt, mc, lc));
  if (mo.shared_ff) {
    RowsGemm gu{h, b->wgu, nullptr, w.sact, M, 2 * mo.shared_ff, H, H, mo.shared_ff, mo.act, mo.shared_limit};
    if (listed_tc<T>(c, M, 2 * mo.shared_ff, H)) RC((listed_gemm_tc<T, TCE_SWIGLU>(c, h, b->wgu, nullptr, w.sact, M, 2 * mo.shared_ff, H, mo.act, mo.shared_ff, mo.shared_limit)));
    else RC((gemm_rows_T<T, RE_GATE_UP>(c, gu)));
    RowsGemm gd{w.sact, b->wd, out, out, M, H, mo.shared_ff, mo.shared_ff, H, 0, 0.f, w.sgate};
    if (listed_tc<T>(c, M, H, mo.shared_ff) && ((uintptr_t)out & 15) == 0) {
      TcExtra xs;
      xs.row_scale = w.sgate;
      RC((listed_gemm_tc<T, TCE_RESIDUAL_F32>(c, w.sact, b->wd, out, out, M, H, mo.shared_ff, 0, 0, 0.f, xs)));
    } else RC((gemm_rows_T<T, RE_RESIDUAL_F32>(c, gd)));
  }
  return CAKE_B200_OK;
}

// x_in, x_out: [B, S, hidden] fp32 (may alias)
static int enqueue_mixer_layers(cake_b200_ctx *c, cake_b200_block *const *blocks, const int *block_idx, int n, cake_b200_cache *kc,
                                const float *x_in, float *x_out, int B, int S, int pos0) {
  const int H = c->cfg.hidden, M = B * S, dt = c->cfg.dtype;
  size_t need = 0;
  for (int i = 0; i < n; i++) {
    need = std::max(need, blocks[i]->ext ? ext_scratch(c, blocks[i], (size_t)M, nullptr, S, pos0 + S).total
                                         : mixer_scratch(c, blocks[i], (size_t)M, nullptr, S, pos0 + S).total);
    if (blocks[i]->m_cos && pos0 + S > blocks[i]->m_rope_rows)
      return fail(CAKE_B200_ESTATE, "position %d exceeds the rotation table (%d rows = the ctx's max_seq)", pos0 + S, blocks[i]->m_rope_rows);
  }
  if (need > c->mx_ws_cap) {
    CU(cudaStreamSynchronize(c->stream));
    if (c->mx_ws) cudaFree(c->mx_ws);
    c->mx_ws = nullptr;
    c->mx_ws_cap = 0;
    CU(cudaMalloc(&c->mx_ws, need));
    c->mx_ws_cap = need;
  }
  cudaStream_t st = c->stream;
  uint64_t *lc = c->capturing ? &c->g_kernels : &c->launches;
  return DISPATCH_T3(dt, T_LAMBDA {
    typedef typename decltype(tag_)::type T;
    const float *cur = x_in;
    for (int i = 0; i < n; i++) {
      const cake_b200_block *b = blocks[i];
      const cake_b200_mixer_spec &sp = b->ms;
      const int l = block_idx[i], inner = sp.heads * sp.vdim;
      if (b->ext) {
        RC(enqueue_ext_layer<T>(c, b, l, kc, cur, x_out, B, S, pos0, lc));
        cur = x_out;
        continue;
      }
      const MixerScratch w = mixer_scratch(c, b, (size_t)M, (char *)c->mx_ws, S, pos0 + S);
      // 1. h = norm1(x); every input projection of the mixer in one product
      RC(launch_pdl(c, norm_shift_rows_kernel<T>, dim3(M), dim3(256), 0, cur, (const int *)nullptr, 1, 0, (const T *)b->ln1, 1, (const T *)nullptr,
                    (const float *)nullptr, (float *)nullptr, (T *)w.h, (T *)nullptr, S, H, c->cfg.rms_eps, pos0, 0.f));
      RowsGemm gi{w.h, b->w_in, nullptr, w.proj, M, b->n_in, H, H, b->n_in_pad, 0, 0.f};
      if (listed_tc<T>(c, M, b->n_in_pad, H)) RC((listed_gemm_tc<T, TCE_PLAIN>(c, w.h, b->w_in, nullptr, w.proj, M, b->n_in_pad, H, 0, 0)));
      else RC((gemm_rows_T<T, RE_STORE>(c, gi)));
      // 2. the mixer: [M, inner] in D
      if (sp.kind == CAKE_B200_MIX_LATENT) {
        const int Dk = sp.kv_rank + sp.rot_dim, qw = sp.dim + sp.rot_dim;
        const int cap_t = latent_cap_t(kc->cap);
        mx::LatentPrep lp{w.proj, b->n_in_pad, sp.heads * qw, b->m_dkv_norm, b->m_cos, b->m_sin, sp.rot.dims, kc->k[l], kc->v[l], cap_t, w.qa,
                          B, S, sp.heads, sp.dim, sp.rot_dim, sp.kv_rank, kc->cap, pos0, c->cfg.rms_eps};
        MX(mx::latent_prep(st, dt, lp, lc));
        // the unrotated query through the key expansion: qa[m, h, :rank] = q[m, h, :dim] . uk[h]   (uk[h]: [dim, rank])
        // long steps in 16-bit D: one tensor-core product per head on column ranges of the step's buffers
        const bool heads_tc = b->m_ukt && M >= 512 && sp.dim % TC_BK == 0 && sp.vdim % TC_BN == 0 && qw % 8 == 0;
        mx::HeadGemm ga{w.proj, b->m_uk, w.qa, M, sp.kv_rank, sp.dim, sp.heads, qw, (long)sp.dim * sp.kv_rank, Dk, b->n_in_pad, sp.kv_rank, sp.heads * Dk, 1};
        if (heads_tc) {
          TcExtra xa;
          xa.a_ld = b->n_in_pad;
          for (int hh = 0; hh < sp.heads; hh++)
            RC((listed_gemm_tc<T, TCE_PLAIN>(c, (const T *)w.proj + (size_t)hh * qw, (const T *)b->m_ukt + (size_t)hh * sp.kv_rank * sp.dim, nullptr,
                                             (T *)w.qa + (size_t)hh * Dk, M, sp.kv_rank, sp.dim, 0, sp.heads * Dk, 0.f, xa)));
        } else MX(mx::head_gemm(st, dt, ga, lc));
        if (w.scores && kc->v[l]) {
          // blocks of lat_tok tokens x heads rows: scores = qa . cache^T on the keys the block's last token sees, softmax with
          // the causal mask into w_hi | w_lo, lat = [w_hi | w_lo] . latent^T with the latent's k coordinate wrapping at kp
          for (int bb = 0; bb < B; bb++)
            for (int t0 = 0; t0 < S; t0 += w.lat_tok) {
              const int nt = std::min(w.lat_tok, S - t0), rows = nt * sp.heads, nk = pos0 + t0 + nt, kp = round_up(nk, TC_BN);
              const T *qa_b = (const T *)w.qa + ((size_t)bb * S + t0) * sp.heads * Dk;
              const T *kc_b = (const T *)kc->k[l] + (size_t)bb * kc->cap * Dk;
              const T *ct_b = (const T *)kc->v[l] + (size_t)bb * sp.kv_rank * cap_t;
              TcExtra xs;
              xs.w_rows = nk;   // rows past the visible keys read as zeros
              RC((listed_gemm_tc<T, TCE_SOFTCAP_F32>(c, qa_b, kc_b, nullptr, w.scores, rows, kp, Dk, 0, 0, 0.f, xs)));
              mx::LatentSoftmax sm{w.scores, w.pw, nt, sp.heads, kp, pos0 + t0, sp.scale};
              MX(mx::latent_softmax(st, dt, sm, lc));
              TcExtra xv;
              xv.b_kwrap = kp;
              xv.w_cols = nk;
              xv.w_ld = cap_t;
              RC((listed_gemm_tc<T, TCE_PLAIN>(c, w.pw, ct_b, nullptr, (T *)w.lat + ((size_t)bb * S + t0) * sp.heads * sp.kv_rank, rows, sp.kv_rank,
                                               2 * kp, 0, 0, 0.f, xv)));
            }
        } else {
          mx::LatentAttn la{w.qa, kc->k[l], w.lat, B, S, sp.heads, sp.kv_rank, sp.rot_dim, kc->cap, pos0, sp.scale, w.part, w.nsplit};
          MX(mx::latent_attention(st, dt, la, lc));
        }
        // the weighted latent through the value expansion: att[m, h, :] = uv[h] lat[m, h]   (uv[h]: [vdim, rank])
        mx::HeadGemm gv{w.lat, b->m_uv, w.att, M, sp.vdim, sp.kv_rank, sp.heads, sp.kv_rank, (long)sp.vdim * sp.kv_rank, sp.vdim,
                        sp.heads * sp.kv_rank, sp.kv_rank, inner, 0};
        if (heads_tc) {
          TcExtra xa;
          xa.a_ld = sp.heads * sp.kv_rank;
          for (int hh = 0; hh < sp.heads; hh++)
            RC((listed_gemm_tc<T, TCE_PLAIN>(c, (const T *)w.lat + (size_t)hh * sp.kv_rank, (const T *)b->m_uv + (size_t)hh * sp.vdim * sp.kv_rank, nullptr,
                                             (T *)w.att + (size_t)hh * sp.vdim, M, sp.vdim, sp.kv_rank, 0, inner, 0.f, xa)));
        } else MX(mx::head_gemm(st, dt, gv, lc));
      } else if (sp.kind == CAKE_B200_MIX_RETENTION) {
        const int qk = sp.heads * sp.dim;
        const T *pj = (const T *)w.proj;
        mx::Recurrence r{pj, pj + qk, pj + 2 * qk, b->n_in_pad, b->n_in_pad, b->n_in_pad, 1, nullptr, 0, nullptr, nullptr, nullptr, b->m_decay,
                         1.0f / sqrtf((float)sp.dim), b->m_cos, b->m_sin, sp.rot.dims, kc->rec_state[l], w.o32, B, S, sp.heads, sp.dim, sp.vdim, pos0};
        MX(mx::recurrence(st, dt, r, lc));
        mx::GateNorm gn{w.o32, pj + 2 * qk + inner, b->n_in_pad, nullptr, w.att, M, inner, sp.heads, 0, c->cfg.rms_eps};
        MX(mx::gate_norm(st, dt, gn, lc));
      } else {
        const int gn_ = sp.groups * sp.state, ch = inner + 2 * gn_;
        const T *pj = (const T *)w.proj, *cv = (const T *)w.conv;
        mx::ShortConv sc{pj, b->n_in_pad, inner, b->m_conv, b->m_conv_b, kc->conv_hist[l], w.conv, B, S, ch, sp.conv, pos0};
        MX(mx::short_conv(st, dt, sc, lc));
        mx::Recurrence r{cv + inner + gn_, cv + inner, cv, ch, ch, ch, sp.heads / sp.groups, pj + inner + ch, b->n_in_pad, b->m_dt_bias, b->m_a_log, b->m_d,
                         nullptr, 1.0f, nullptr, nullptr, 0, kc->rec_state[l], w.o32, B, S, sp.heads, sp.state, sp.vdim, pos0};
        MX(mx::recurrence(st, dt, r, lc));
        mx::GateNorm gn{w.o32, pj, b->n_in_pad, b->m_norm, w.att, M, inner, sp.norm_groups, 1, c->cfg.rms_eps};
        MX(mx::gate_norm(st, dt, gn, lc));
      }
      // 3. x <- x + o(att)
      RowsGemm go{w.att, b->wo, cur, x_out, M, H, inner, inner, H, 0, 0.f};
      if (listed_tc<T>(c, M, H, inner) && (((uintptr_t)cur | (uintptr_t)x_out) & 15) == 0)
        RC((listed_gemm_tc<T, TCE_RESIDUAL_F32>(c, w.att, b->wo, cur, x_out, M, H, inner, 0, 0)));
      else RC((gemm_rows_T<T, RE_RESIDUAL_F32>(c, go)));
      cur = x_out;
      // 4. x <- x + routed experts(norm2(x)) + gate * shared expert
      if (sp.moe.experts + sp.moe.identity > 0) {
        RC(launch_pdl(c, norm_shift_rows_kernel<T>, dim3(M), dim3(256), 0, cur, (const int *)nullptr, 1, 0, (const T *)b->ln2, 1, (const T *)nullptr,
                      (const float *)nullptr, (float *)nullptr, (T *)w.h, (T *)nullptr, S, H, c->cfg.rms_eps, pos0, 0.f));
        RC(enqueue_routed_ff<T>(c, b, w.moe, w.h, cur, x_out, M, lc));
      }
    }
    return CAKE_B200_OK;
  });
}

extern "C" int cake_b200_stream_inject(cake_b200_ctx *c, float *x_dev, const float *x0_dev, const void *vec, int slot, int rows) {
  if (!c || !x_dev || !vec || rows < 1 || slot < 0 || slot >= 64) return fail(CAKE_B200_EINVAL, "bad stream_inject arguments");
  if (!c->cfg.layer_list) return fail(CAKE_B200_EINVAL, "stream_inject is for models with an fp32 residual stream");
  CU(cudaSetDevice(c->device));
  if (c->inject_src[slot] != vec) {
    if (c->inject_vec[slot]) { CU(cudaStreamSynchronize(c->stream)); cudaFree(c->inject_vec[slot]); c->inject_vec[slot] = nullptr; }
    RC(upload(c, &c->inject_vec[slot], vec, (size_t)c->cfg.hidden * c->es));
    RC(pipe_mark(c));
    c->inject_src[slot] = vec;
  }
  RC(wait_loads(c));
  MX(mx::stream_inject(c->stream, c->cfg.dtype, x_dev, x0_dev, c->inject_vec[slot], rows, c->cfg.hidden, &c->launches));
  return CAKE_B200_OK;
}

extern "C" int cake_b200_stream_project(cake_b200_ctx *c, float *x_dev, const float *x0_dev, const void *w, int rows) {
  if (!c || !x_dev || !x0_dev || !w || rows < 1) return fail(CAKE_B200_EINVAL, "bad stream_project arguments");
  if (!c->cfg.layer_list) return fail(CAKE_B200_EINVAL, "stream_project is for models with an fp32 residual stream");
  CU(cudaSetDevice(c->device));
  const size_t H = c->cfg.hidden;
  if (c->proj_src != w) {
    if (c->proj_w) { CU(cudaStreamSynchronize(c->stream)); cudaFree(c->proj_w); c->proj_w = nullptr; }
    RC(upload(c, &c->proj_w, w, H * 2 * H * c->es));
    RC(pipe_mark(c));
    c->proj_src = w;
  }
  RC(wait_loads(c));
  const size_t need = (size_t)rows * 2 * H * c->es + 16;
  if (need > c->proj_ws_cap) {
    CU(cudaStreamSynchronize(c->stream));
    if (c->proj_ws) cudaFree(c->proj_ws);
    c->proj_ws = nullptr;
    c->proj_ws_cap = 0;
    CU(cudaMalloc(&c->proj_ws, need));
    c->proj_ws_cap = need;
  }
  MX(mx::concat_rows(c->stream, c->cfg.dtype, x_dev, x0_dev, c->proj_ws, rows, (int)H, &c->launches));
  return DISPATCH_T3(c->cfg.dtype, T_LAMBDA {
    typedef typename decltype(tag_)::type T;
    return gemm_f32_out<T>(c, c->proj_ws, c->proj_w, x_dev, rows, (int)H, 2 * (int)H);
  });
}

// ------------------------------------------------------------------------------------------ forward_batch
extern "C" int cake_b200_forward_batch(cake_b200_ctx *c, cake_b200_block *const *blocks, const int *block_idx,
                                       int n_blocks, cake_b200_cache *kc, const void *x_dev, void *y_dev, int batch,
                                       int seq, int index_pos) {
  if (!c || !blocks || !block_idx || !kc || !x_dev || !y_dev || n_blocks < 1) return fail(CAKE_B200_EINVAL, "null/empty argument");
  if (batch != kc->batch) return fail(CAKE_B200_EINVAL, "batch %d != cache batch %d", batch, kc->batch);
  if (seq < 1 || index_pos < 0 || (long long)index_pos + (long long)seq > (long long)kc->cap)
    return fail(CAKE_B200_ESTATE, "index_pos %d + seq %d exceeds cache capacity %d", index_pos, seq, kc->cap);
  CU(cudaSetDevice(c->device));
  RC(wait_loads(c));
  bool listed = false, mixer = false;
  for (int i = 0; i < n_blocks; i++) {
    if (!blocks[i]) return fail(CAKE_B200_EINVAL, "blocks[%d] is null", i);
    listed = listed || blocks[i]->listed;
    mixer = mixer || blocks[i]->mixer;
    if (blocks[i]->listed != listed || blocks[i]->mixer != mixer) return fail(CAKE_B200_EINVAL, "blocks of different families cannot share a call");
  }
  for (int i = 0; i < n_blocks; i++) {
    if (mixer) RC(cache_ensure_mixer(kc, block_idx[i], blocks[i]));
    else if (listed) RC(cache_ensure_listed(kc, block_idx[i], blocks[i]));
    else RC(cache_ensure(kc, block_idx[i]));
    if (kc->len[block_idx[i]] != index_pos)
      return fail(CAKE_B200_ESTATE, "block %d: index_pos %d != cache length %d (clear the cache or feed positions in order)",
                  block_idx[i], index_pos, kc->len[block_idx[i]]);
  }
  if (mixer) {  // fp32 residual stream
    RC(enqueue_mixer_layers(c, blocks, block_idx, n_blocks, kc, (const float *)x_dev, (float *)y_dev, batch, seq, index_pos));
    for (int i = 0; i < n_blocks; i++) kc->len[block_idx[i]] = index_pos + seq;
    CU(cudaGetLastError());
    return CAKE_B200_OK;
  }
  if (listed) {  // fp32 residual stream: x_dev / y_dev are float
    RC(enqueue_listed_layers(c, blocks, block_idx, n_blocks, kc, (const float *)x_dev, (float *)y_dev, batch, seq, index_pos));
    for (int i = 0; i < n_blocks; i++) {
      kc->len[block_idx[i]] = index_pos + seq;
      if (blocks[i]->shift) kc->shift_cur[block_idx[i]] ^= 1;
    }
    CU(cudaGetLastError());
    return CAKE_B200_OK;
  }
  bool variant = false;  // sibling block structures step through the batched path (cake_b200_block_set_variant)
  for (int i = 0; i < n_blocks; i++) {
    if (!blocks[i]) return fail(CAKE_B200_EINVAL, "blocks[%d] is null", i);
    variant = variant || blocks[i]->variant();
  }
  if (batch == 1 && seq == 1 && !variant) {
    set_int_kernel<<<1, 1, 0, c->stream>>>(kc->d_pos, index_pos);
    c->launches++;
    if (c->use_mega && mega_supported(c)) RC(enqueue_mega_layers(c, blocks, block_idx, n_blocks, kc, x_dev, y_dev));
    else RC(enqueue_decode_layers(c, blocks, block_idx, n_blocks, kc, x_dev, y_dev));
  } else {
    RC(enqueue_prefill_layers(c, blocks, block_idx, n_blocks, kc, x_dev, y_dev, batch, seq, index_pos));
  }
  for (int i = 0; i < n_blocks; i++) kc->len[block_idx[i]] = index_pos + seq;
  CU(cudaGetLastError());
  return CAKE_B200_OK;
}

static int io_reserve(cake_b200_ctx *c, size_t bytes) {
  if (bytes > c->io_x_cap) {
    CU(cudaStreamSynchronize(c->stream));
    if (c->io_x) cudaFree(c->io_x);
    CU(cudaMalloc(&c->io_x, bytes));
    c->io_x_cap = bytes;
  }
  if (bytes > c->h_pin_x_cap) {
    if (c->h_pin_x) cudaFreeHost(c->h_pin_x);
    CU(cudaMallocHost(&c->h_pin_x, bytes));
    c->h_pin_x_cap = bytes;
  }
  return CAKE_B200_OK;
}

extern "C" int cake_b200_forward_batch_host(cake_b200_ctx *c, cake_b200_block *const *blocks, const int *block_idx,
                                            int n_blocks, cake_b200_cache *kc, const void *x_host, void *y_host,
                                            int batch, int seq, int index_pos) {
  if (!c || !x_host || !y_host || !kc) return fail(CAKE_B200_EINVAL, "null argument");
  // validated BEFORE any size is derived from them: the dims may come off the wire (cake_worker)
  if (batch < 1 || seq < 1 || batch != kc->batch) return fail(CAKE_B200_EINVAL, "batch %d (cache batch %d) / seq %d out of range", batch, kc->batch, seq);
  if (index_pos < 0 || (long long)index_pos + (long long)seq > (long long)kc->cap)
    return fail(CAKE_B200_ESTATE, "index_pos %d + seq %d exceeds cache capacity %d", index_pos, seq, kc->cap);
  CU(cudaSetDevice(c->device));
  const size_t bytes = (size_t)batch * seq * c->cfg.hidden * (c->cfg.layer_list ? sizeof(float) : c->es);
  RC(io_reserve(c, bytes));
  memcpy(c->h_pin_x, x_host, bytes);
  CU(cudaMemcpyAsync(c->io_x, c->h_pin_x, bytes, cudaMemcpyHostToDevice, c->stream));
  RC(cake_b200_forward_batch(c, blocks, block_idx, n_blocks, kc, c->io_x, c->io_x, batch, seq, index_pos));
  CU(cudaMemcpyAsync(c->h_pin_x, c->io_x, bytes, cudaMemcpyDeviceToHost, c->stream));
  CU(cudaStreamSynchronize(c->stream));
  memcpy(y_host, c->h_pin_x, bytes);
  return CAKE_B200_OK;
}

// ------------------------------------------------------------------------------------------ head / tail
extern "C" int cake_b200_head_load(cake_b200_ctx *c, const void *embed, const void *ln_f, const void *lm_head) {
  if (!c || !embed || !ln_f) return fail(CAKE_B200_EINVAL, "null argument");
  if (!lm_head && !c->cfg.tie_embeddings) return fail(CAKE_B200_EINVAL, "lm_head is NULL but tie_embeddings is 0");
  CU(cudaSetDevice(c->device));
  const size_t es = c->es, H = c->cfg.hidden, V = c->cfg.vocab;
  RC(upload(c, &c->embed, embed, V * H * es));
  RC(upload(c, &c->ln_f, ln_f, (c->cfg.layer_list && c->cfg.scalar_final_norm ? 1 : H) * es));
  if (lm_head) RC(upload(c, &c->lm_head, lm_head, V * H * es));
  else c->lm_head = c->embed;  // text_model.rs:164-167
  return pipe_mark(c);
}

extern "C" int cake_b200_embed(cake_b200_ctx *c, const uint32_t *ids_host, int batch, int seq, void *x_dev) {
  if (!c || !ids_host || !x_dev || !c->embed) return fail(CAKE_B200_EINVAL, "null argument or head not loaded");
  CU(cudaSetDevice(c->device));
  RC(wait_loads(c));
  if (batch < 1 || seq < 1) return fail(CAKE_B200_EINVAL, "embed: batch and seq must be >= 1");
  const size_t n = (size_t)batch * seq;
  for (size_t i = 0; i < n; i++)  // index_select on an out-of-range id is an error in the reference (backends/mod.rs:513-528)
    if (ids_host[i] >= (uint32_t)c->cfg.vocab)
      return fail(CAKE_B200_EINVAL, "token id %u at %zu out of range (vocab %d)", ids_host[i], i, c->cfg.vocab);
  if (n > c->d_ids_cap) {
    CU(cudaStreamSynchronize(c->stream));
    if (c->d_ids) cudaFree(c->d_ids);
    CU(cudaMalloc(&c->d_ids, n * 4));
    c->d_ids_cap = n;
  }
  CU(cudaMemcpyAsync(c->d_ids, ids_host, n * 4, cudaMemcpyHostToDevice, c->stream));
  c->d_ids_n = n;
  // the ids buffer is pageable in general: the copy above returns after staging, safe to reuse
  if (c->cfg.layer_list)  // the fp32 residual stream starts here
    return DISPATCH_T3(c->cfg.dtype, T_LAMBDA {
      typedef typename decltype(tag_)::type T;
      return launch_pdl(c, embed_f32_kernel<T>, dim3((unsigned)n), dim3(128), 0, (const T *)c->embed, (const uint32_t *)c->d_ids,
                        (float *)x_dev, (int)n, c->cfg.hidden, c->cfg.vocab, c->cfg.embed_scale);
    });
  RC(DISPATCH_T(c->cfg.dtype, T_LAMBDA {
      typedef typename decltype(tag_)::type T;
    return launch_pdl(c, embed_kernel<T>, dim3((unsigned)n), dim3(128), 0, (const T *)c->embed, (const uint32_t *)c->d_ids,
                      (T *)x_dev, (int)n, c->cfg.hidden, c->cfg.vocab, c->cfg.embed_scale);
  }));
  return CAKE_B200_OK;
}


extern "C" int cake_b200_head_load_tables(cake_b200_ctx *c, const cake_b200_embed_tables *t) {
  if (!c || !t) return fail(CAKE_B200_EINVAL, "null argument");
  if (!c->cfg.layer_list) return fail(CAKE_B200_EINVAL, "head_load_tables is for models with an fp32 residual stream");
  if ((t->bigram && (t->bigram_rows < 2 || t->mul_prev < 0 || t->mul_cur < 0)) || (t->pos && t->pos_rows < 1)) return fail(CAKE_B200_EINVAL, "bad embedding table sizes");
  CU(cudaSetDevice(c->device));
  const size_t H = c->cfg.hidden;
  if (t->bigram) {
    RC(upload(c, &c->bigram, t->bigram, (size_t)t->bigram_rows * H * c->es));
    c->bigram_rows = t->bigram_rows;
    c->mul_prev = t->mul_prev;
    c->mul_cur = t->mul_cur;
  }
  if (t->pos) {
    RC(upload(c, &c->pos_tab, t->pos, (size_t)t->pos_rows * H * c->es));
    c->pos_rows = t->pos_rows;
  }
  c->final_norm_offset = t->final_norm_offset;
  if (t->side) {
    if (t->side_cols < 1) return fail(CAKE_B200_EINVAL, "bad side table size");
    RC(upload(c, &c->side_tab, t->side, (size_t)c->cfg.vocab * t->side_cols * c->es));
    c->side_cols = t->side_cols;
  }
  if (t->final_norm_kind == 1) {
    if (!t->final_bias || c->cfg.scalar_final_norm) return fail(CAKE_B200_EINVAL, "the squashing final norm needs its offset vector and a vector gain");
    RC(upload(c, &c->ln_f_b, t->final_bias, H * c->es));
    c->final_norm_kind = 1;
    c->final_alpha = t->final_alpha;
  } else if (t->final_norm_kind != 0) return fail(CAKE_B200_EINVAL, "final_norm_kind %d", t->final_norm_kind);
  return pipe_mark(c);
}

extern "C" int cake_b200_embed_at(cake_b200_ctx *c, cake_b200_cache *kc, const uint32_t *ids_host, int batch, int seq, int index_pos, void *x_dev) {
  if (!c || !kc || !ids_host || !x_dev || !c->embed) return fail(CAKE_B200_EINVAL, "null argument or head not loaded");
  if (!c->cfg.layer_list) return fail(CAKE_B200_EINVAL, "embed_at is for models with an fp32 residual stream");
  if (batch < 1 || seq < 1 || batch != kc->batch) return fail(CAKE_B200_EINVAL, "embed_at: batch %d (cache batch %d) / seq %d", batch, kc ? kc->batch : 0, seq);
  if (index_pos != kc->embed_len) return fail(CAKE_B200_ESTATE, "embed_at: index_pos %d != the position %d the embedding has reached in this cache", index_pos, kc->embed_len);
  if (c->pos_tab && index_pos + seq > c->pos_rows) return fail(CAKE_B200_ESTATE, "position %d exceeds the %d learned positions", index_pos + seq, c->pos_rows);
  CU(cudaSetDevice(c->device));
  RC(wait_loads(c));
  const size_t n = (size_t)batch * seq;
  for (size_t i = 0; i < n; i++)
    if (ids_host[i] >= (uint32_t)c->cfg.vocab) return fail(CAKE_B200_EINVAL, "token id %u at %zu out of range (vocab %d)", ids_host[i], i, c->cfg.vocab);
  if (n + batch > c->d_ids_cap) {
    CU(cudaStreamSynchronize(c->stream));
    if (c->d_ids) cudaFree(c->d_ids);
    c->d_ids = nullptr;
    c->d_ids_cap = 0;
    CU(cudaMalloc(&c->d_ids, (n + batch) * 4));
    c->d_ids_cap = n + batch;
  }
  CU(cudaMemcpyAsync(c->d_ids, ids_host, n * 4, cudaMemcpyHostToDevice, c->stream));
  CU(cudaMemcpyAsync(c->d_ids + n, kc->last_tok.data(), (size_t)batch * 4, cudaMemcpyHostToDevice, c->stream));
  c->d_ids_n = n;
  CU(cudaStreamSynchronize(c->stream));  // both sources are pageable host memory that changes below / belongs to the caller
  mx::EmbedTables et{c->embed, c->d_ids, c->bigram, c->pos_tab, (float *)x_dev, batch, seq, c->cfg.hidden, c->cfg.vocab, c->bigram_rows - 1,
                     c->mul_prev, c->mul_cur, index_pos, c->cfg.embed_scale};
  MX(mx::embed_tables(c->stream, c->cfg.dtype, et, &c->launches));
  for (int b = 0; b < batch; b++) kc->last_tok[b] = ids_host[(size_t)b * seq + seq - 1];
  kc->embed_len = index_pos + seq;
  return CAKE_B200_OK;
}

// fp32 logits of n rows of the fp32 stream: final norm (scalar or vector gain) -> lm_head -> soft cap
// rows_host == NULL: row i = i * row_mul + row_add (no table, nothing to wait for)
static int listed_logits(cake_b200_ctx *c, const void *x_dev, const int *rows_host, int row_mul, int row_add, int n, float *out_dev) {
  const size_t H = c->cfg.hidden, V = c->cfg.vocab;
  if ((size_t)n > c->sp_logit_rows) {
    CU(cudaStreamSynchronize(c->stream));
    if (c->sp_hn) cudaFree(c->sp_hn);
    if (c->sp_rows_idx) cudaFree(c->sp_rows_idx);
    if (c->sp_logits) cudaFree(c->sp_logits);
    c->sp_hn = nullptr; c->sp_rows_idx = nullptr; c->sp_logits = nullptr; c->sp_logit_rows = 0;
    CU(cudaMalloc(&c->sp_hn, (size_t)n * H * c->es + 16));
    CU(cudaMalloc(&c->sp_rows_idx, (size_t)n * sizeof(int)));
    CU(cudaMalloc(&c->sp_logits, (size_t)n * V * sizeof(float)));
    c->sp_logit_rows = n;
  }
  if (rows_host) {
    CU(cudaMemcpyAsync(c->sp_rows_idx, rows_host, (size_t)n * sizeof(int), cudaMemcpyHostToDevice, c->stream));
    CU(cudaStreamSynchronize(c->stream));  // rows_host is the caller's (pageable) memory
  }
  return DISPATCH_T3(c->cfg.dtype, T_LAMBDA {
    typedef typename decltype(tag_)::type T;
    if (c->final_norm_kind == 1) {
      mx::TanhNorm fn{(const float *)x_dev, rows_host ? c->sp_rows_idx : nullptr, row_mul, row_add, c->ln_f, c->ln_f_b, c->final_alpha, nullptr, nullptr,
                      c->sp_hn, n, (int)H};
      MX(mx::tanh_norm(c->stream, c->cfg.dtype, fn, &c->launches));
    } else
    RC(launch_pdl(c, norm_shift_rows_kernel<T>, dim3(n), dim3(256), 0, (const float *)x_dev, (const int *)(rows_host ? c->sp_rows_idx : nullptr),
                  row_mul, row_add, (const T *)c->ln_f,
                  c->cfg.scalar_final_norm ? 0 : 1, (const T *)nullptr, (const float *)nullptr, (float *)nullptr, (T *)c->sp_hn, (T *)nullptr, 1,
                  (int)H, c->cfg.rms_eps, 0, c->final_norm_offset));
    RowsGemm g{c->sp_hn, c->lm_head, nullptr, out_dev ? out_dev : c->sp_logits, n, (int)V, (int)H, (int)H, (int)V, 0, c->cfg.logit_softcap};
    if (listed_tc<T>(c, n, (int)V, (int)H))
      return listed_gemm_tc<T, TCE_SOFTCAP_F32>(c, c->sp_hn, c->lm_head, nullptr, g.C, n, (int)V, (int)H, 0, 0, c->cfg.logit_softcap);
    return gemm_rows_T<T, RE_SOFTCAP_F32>(c, g);
  });
}
// cake_b200_logits for a layer-list model: the last position of every batch row; logits_dev receives them in the 16-bit
// dtype the samplers read (bf16 when D is fp32)
static int listed_logits_last(cake_b200_ctx *c, const void *x_dev, int batch, int seq, void *logits_dev, uint32_t *argmax_host) {
  RC(listed_logits(c, x_dev, nullptr, seq, seq - 1, batch, nullptr));
  const size_t V = c->cfg.vocab;
  if (!logits_dev && !argmax_host) return CAKE_B200_OK;
  return DISPATCH_T(c->cfg.dtype, T_LAMBDA {
    typedef typename decltype(tag_)::type T;
    if (logits_dev) RC(launch_pdl(c, f32_to_T_kernel<T>, dim3(64), dim3(256), 0, (const float *)c->sp_logits, (T *)logits_dev, (size_t)batch * V));
    if (argmax_host) {
      for (int b = 0; b < batch; b++) {
        T *row = logits_dev ? (T *)logits_dev + (size_t)b * V : (T *)c->logits;
        if (!logits_dev) RC(launch_pdl(c, f32_to_T_kernel<T>, dim3(64), dim3(256), 0, (const float *)c->sp_logits + (size_t)b * V, row, V));
        argmax_kernel<T><<<1, 1024, 0, c->stream>>>(row, (int)V, c->d_token);
        c->launches++;
        CU(cudaMemcpyAsync(c->h_pin + b, c->d_token, 4, cudaMemcpyDeviceToHost, c->stream));
      }
      CU(cudaStreamSynchronize(c->stream));
      for (int b = 0; b < batch; b++) argmax_host[b] = c->h_pin[b];
    }
    return CAKE_B200_OK;
  });
}
extern "C" int cake_b200_logits_rows(cake_b200_ctx *c, const void *x_dev, int n_rows_total, const int *rows_host, int n,
                                     float *logits_f32_dev) {
  if (!c || !x_dev || !rows_host || !logits_f32_dev || !c->lm_head) return fail(CAKE_B200_EINVAL, "null argument or head not loaded");
  if (!c->cfg.layer_list) return fail(CAKE_B200_EINVAL, "logits_rows is for layer-list models (fp32 residual stream)");
  if (n < 1) return fail(CAKE_B200_EINVAL, "logits_rows: n must be >= 1");
  for (int i = 0; i < n; i++)
    if (rows_host[i] < 0 || rows_host[i] >= n_rows_total) return fail(CAKE_B200_EINVAL, "row %d out of range (%d rows)", rows_host[i], n_rows_total);
  CU(cudaSetDevice(c->device));
  RC(wait_loads(c));
  return listed_logits(c, x_dev, rows_host, 1, 0, n, logits_f32_dev);
}

extern "C" int cake_b200_logits(cake_b200_ctx *c, const void *x_dev, int batch, int seq, void *logits_dev,
                                uint32_t *argmax_host) {
  if (!c || !x_dev || !c->lm_head) return fail(CAKE_B200_EINVAL, "null argument or head not loaded");
  if (batch > 64) return fail(CAKE_B200_EINVAL, "batch > 64");
  CU(cudaSetDevice(c->device));
  RC(wait_loads(c));
  if (c->cfg.layer_list) return listed_logits_last(c, x_dev, batch, seq, logits_dev, argmax_host);
  const size_t H = c->cfg.hidden, V = c->cfg.vocab, es = c->es;
  for (int b = 0; b < batch; b++) {
    const char *row = (const char *)x_dev + ((size_t)b * seq + (seq - 1)) * H * es;  // text_model.rs:342-346
    void *lo = logits_dev ? (char *)logits_dev + (size_t)b * V * es : c->logits;
    RC(enqueue_head(c, row, lo, false));
    if (argmax_host) CU(cudaMemcpyAsync(c->h_pin + b, c->d_token, 4, cudaMemcpyDeviceToHost, c->stream));
  }
  if (argmax_host) {
    CU(cudaStreamSynchronize(c->stream));
    for (int b = 0; b < batch; b++) argmax_host[b] = c->h_pin[b];
  }
  return CAKE_B200_OK;
}

static int apply_repeat_penalty(cake_b200_ctx *c, void *logits_dev, float penalty, const uint32_t *ctx_tokens_host, int n_tokens);
extern "C" int cake_b200_repeat_penalty_argmax(cake_b200_ctx *c, void *logits_dev, float penalty,
                                               const uint32_t *ctx_tokens_host, int n_tokens, uint32_t *argmax_host) {
  if (!c || !logits_dev || !argmax_host) return fail(CAKE_B200_EINVAL, "null argument");
  CU(cudaSetDevice(c->device));
  RC(apply_repeat_penalty(c, logits_dev, penalty, ctx_tokens_host, n_tokens));
  RC(DISPATCH_T(c->cfg.dtype, T_LAMBDA {
      typedef typename decltype(tag_)::type T;
    argmax_kernel<T><<<1, 1024, 0, c->stream>>>((const T *)logits_dev, c->cfg.vocab, c->d_token);
    return CAKE_B200_OK;
  }));
  c->launches++;
  CU(cudaMemcpyAsync(c->h_pin, c->d_token, 4, cudaMemcpyDeviceToHost, c->stream));
  CU(cudaStreamSynchronize(c->stream));
  *argmax_host = c->h_pin[0];
  return CAKE_B200_OK;
}

// ------------------------------------------------------------------------------------------ samplers (sample.cuh)
static int check_sampling(const cake_b200_ctx *c, const cake_b200_sampling *s) {
  if (s->kind < 0 || s->kind > 5) return fail(CAKE_B200_EINVAL, "sampling kind %d unknown (0..5)", s->kind);
  if ((s->kind == SAMPLE_TOPK || s->kind == SAMPLE_TOPK_TOPP) && (s->top_k < 1 || (s->top_k > SAMPLE_MAX_K && s->top_k < c->cfg.vocab)))
    return fail(CAKE_B200_EINVAL, "top_k %d unsupported (1..%d, or >= vocab)", s->top_k, SAMPLE_MAX_K);
  return CAKE_B200_OK;
}
static int samp_reserve(cake_b200_ctx *c) {
  if (!c->samp_p) CU(cudaMalloc(&c->samp_p, (size_t)c->cfg.vocab * 4 + 16));
  return CAKE_B200_OK;
}
static SampleArgs to_args(const cake_b200_sampling &s) { return SampleArgs{s.kind, s.top_k, s.temperature, s.top_p, (unsigned long long)s.seed}; }

static int apply_repeat_penalty(cake_b200_ctx *c, void *logits_dev, float penalty, const uint32_t *ctx_tokens_host, int n_tokens) {
  // text_model.rs:66-72: de-duplicate, keeping first occurrences
  std::vector<uint32_t> uniq;
  for (int i = 0; i < n_tokens; i++) {
    bool dup = false;
    for (uint32_t u : uniq) dup |= (u == ctx_tokens_host[i]);
    if (!dup) uniq.push_back(ctx_tokens_host[i]);
  }
  if (uniq.empty() || penalty == 1.0f) return CAKE_B200_OK;
  if (uniq.size() > c->d_pen_cap) {
    CU(cudaStreamSynchronize(c->stream));
    if (c->d_pen) cudaFree(c->d_pen);
    CU(cudaMalloc(&c->d_pen, uniq.size() * 4));
    c->d_pen_cap = uniq.size();
  }
  CU(cudaMemcpyAsync(c->d_pen, uniq.data(), uniq.size() * 4, cudaMemcpyHostToDevice, c->stream));
  CU(cudaStreamSynchronize(c->stream));  // uniq is a stack-owned pageable buffer
  RC(DISPATCH_T(c->cfg.dtype, T_LAMBDA {
    typedef typename decltype(tag_)::type T;
    repeat_penalty_kernel<T><<<(unsigned)((uniq.size() + 127) / 128), 128, 0, c->stream>>>((T *)logits_dev, c->cfg.vocab, penalty, c->d_pen, (int)uniq.size());
    return CAKE_B200_OK;
  }));
  c->launches++;
  return CAKE_B200_OK;
}

extern "C" int cake_b200_sample(cake_b200_ctx *c, void *logits_dev, const cake_b200_sampling *s, float repeat_penalty,
                                const uint32_t *ctx_tokens_host, int n_tokens, uint64_t step, const float *noise_host,
                                uint32_t *token_host) {
  if (!c || !logits_dev || !s || !token_host || n_tokens < 0 || (n_tokens > 0 && !ctx_tokens_host)) return fail(CAKE_B200_EINVAL, "null argument");
  RC(check_sampling(c, s));
  CU(cudaSetDevice(c->device));
  RC(samp_reserve(c));
  RC(apply_repeat_penalty(c, logits_dev, repeat_penalty, ctx_tokens_host, n_tokens));
  const float *noise_dev = nullptr;
  if (noise_host) {
    const size_t n = (s->kind == SAMPLE_GUMBEL) ? (size_t)c->cfg.vocab : 1;
    if (!c->samp_noise) CU(cudaMalloc(&c->samp_noise, (size_t)c->cfg.vocab * 4 + 16));
    CU(cudaMemcpyAsync(c->samp_noise, noise_host, n * 4, cudaMemcpyHostToDevice, c->stream));
    CU(cudaStreamSynchronize(c->stream));
    noise_dev = c->samp_noise;
  }
  set_int_kernel<<<1, 1, 0, c->stream>>>((int *)(c->samp_p + c->cfg.vocab), (int)(step & 0x7fffffff));  // the draw's counter
  RC(DISPATCH_T(c->cfg.dtype, T_LAMBDA {
    typedef typename decltype(tag_)::type T;
    sample_kernel<T><<<1, SAMPLE_THREADS, 0, c->stream>>>((const T *)logits_dev, c->cfg.vocab, to_args(*s), c->samp_p, noise_dev,
                                                          (const int *)(c->samp_p + c->cfg.vocab), 0, c->d_token, nullptr, 1);
    return CAKE_B200_OK;
  }));
  c->launches += 2;
  CU(cudaGetLastError());
  CU(cudaMemcpyAsync(c->h_pin, c->d_token, 4, cudaMemcpyDeviceToHost, c->stream));
  CU(cudaStreamSynchronize(c->stream));
  *token_host = c->h_pin[0];
  return CAKE_B200_OK;
}

extern "C" int cake_b200_decode_set_sampling(cake_b200_ctx *c, const cake_b200_sampling *s) {
  if (!c) return fail(CAKE_B200_EINVAL, "null argument");
  if (!s) { c->sampling = cake_b200_sampling{}; return CAKE_B200_OK; }
  RC(check_sampling(c, s));
  CU(cudaSetDevice(c->device));
  RC(samp_reserve(c));  // no allocation inside the graph capture of decode_build
  c->sampling = *s;
  return CAKE_B200_OK;
}

// ------------------------------------------------------------------------------------------ comm
extern "C" int cake_b200_comm_unique_id(void *out128) {
  if (!out128) return fail(CAKE_B200_EINVAL, "null argument");
  RC(nccl_load());
  ncclUniqueId id;
  NC(g_nccl.GetUniqueId(&id));
  static_assert(sizeof(ncclUniqueId) == 128, "ncclUniqueId is 128 bytes");
  memcpy(out128, &id, 128);
  return CAKE_B200_OK;
}
extern "C" int cake_b200_comm_init(cake_b200_ctx *c, const void *unique_id128, int rank, int world) {
  if (!c || !unique_id128 || rank < 0 || rank >= world) return fail(CAKE_B200_EINVAL, "bad comm arguments");
  RC(nccl_load());
  CU(cudaSetDevice(c->device));
  ncclUniqueId id;
  memcpy(&id, unique_id128, 128);
  NC(g_nccl.CommInitRank(&c->comm, world, id, rank));
  c->rank = rank;
  c->world = world;
  // Warm up the ring's p2p connections now: NCCL sets a peer connection up lazily on first use, which must
  // not happen inside the CUDA-graph capture of the decode step.
  if (world > 1) {
    const size_t xbytes = (size_t)c->cfg.hidden * c->es;
    NC(g_nccl.GroupStart());
    NC(g_nccl.Send(c->xa, xbytes, ncclUint8, (rank + 1) % world, c->comm, c->stream));
    NC(g_nccl.Recv(c->xb, xbytes, ncclUint8, (rank + world - 1) % world, c->comm, c->stream));
    NC(g_nccl.GroupEnd());
    CU(cudaStreamSynchronize(c->stream));
  }
  return CAKE_B200_OK;
}
extern "C" int cake_b200_send(cake_b200_ctx *c, const void *x_dev, size_t bytes, int peer) {
  if (!c || !c->comm) return fail(CAKE_B200_ESTATE, "communicator not initialised");
  NC(g_nccl.Send(x_dev, bytes, ncclUint8, peer, c->comm, c->stream));
  return CAKE_B200_OK;
}
extern "C" int cake_b200_recv(cake_b200_ctx *c, void *x_dev, size_t bytes, int peer) {
  if (!c || !c->comm) return fail(CAKE_B200_ESTATE, "communicator not initialised");
  NC(g_nccl.Recv(x_dev, bytes, ncclUint8, peer, c->comm, c->stream));
  return CAKE_B200_OK;
}

// Ring hand-off over NVLink peer memory.  Each rank owns an inbox {u64 arrivals, pad to 128 B, x[hidden]} that the
// previous rank's decode kernel writes directly (st.global over NVLink) and releases with one red.release.sys per CTA.
constexpr size_t INBOX_X_OFF = 128;
extern "C" int cake_b200_ring_export(cake_b200_ctx *c, void *handle64) {
  if (!c || !handle64) return fail(CAKE_B200_EINVAL, "null argument");
  CU(cudaSetDevice(c->device));
  if (!c->inbox) {
    CU(cudaMalloc(&c->inbox, INBOX_X_OFF + (size_t)c->cfg.hidden * c->es + 128));
    CU(cudaMemset(c->inbox, 0, INBOX_X_OFF + (size_t)c->cfg.hidden * c->es + 128));
  }
  cudaIpcMemHandle_t h;
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "cudaIpcMemHandle_t is 64 bytes");
  CU(cudaIpcGetMemHandle(&h, c->inbox));
  memcpy(handle64, &h, 64);
  return CAKE_B200_OK;
}
extern "C" int cake_b200_ring_import(cake_b200_ctx *c, const void *next_rank_handle64) {
  if (!c || !next_rank_handle64) return fail(CAKE_B200_EINVAL, "null argument");
  CU(cudaSetDevice(c->device));
  cudaIpcMemHandle_t h;
  memcpy(&h, next_rank_handle64, 64);
  void *p = nullptr;
  CU(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess));
  c->peer_inbox = (unsigned char *)p;
  return CAKE_B200_OK;
}

// ------------------------------------------------------------------------------------------ decode loop (one CUDA graph per shard)
extern "C" int cake_b200_decode_build(cake_b200_ctx *c, cake_b200_block *const *blocks, const int *block_idx,
                                      int n_blocks, cake_b200_cache *kc, int rank, int world) {
  if (!c || !kc || n_blocks < 0 || world < 1 || rank < 0 || rank >= world) return fail(CAKE_B200_EINVAL, "bad decode_build arguments");
  if (kc->batch != 1) return fail(CAKE_B200_EINVAL, "decode graph is batch 1 (cake run/serve never batch, text_model.rs:418-420)");
  if (world > 1 && !c->comm) return fail(CAKE_B200_ESTATE, "world > 1 needs cake_b200_comm_init first");
  if (rank == 0 && !c->lm_head) return fail(CAKE_B200_ESTATE, "rank 0 needs cake_b200_head_load first");
  for (int i = 0; i < n_blocks; i++)
    if (blocks[i] && blocks[i]->variant())
      return fail(CAKE_B200_EINVAL, "block %d is a sibling block structure (cake_b200_block_set_variant / pre-reshape QK-norm): "
                  "the decode graph covers the standard block only; step it with cake_b200_forward_batch", block_idx[i]);
  CU(cudaSetDevice(c->device));
  RC(wait_loads(c));
  for (int i = 0; i < n_blocks; i++) RC(cache_ensure(kc, block_idx[i]));
  if (c->gexec) { cudaGraphExecDestroy(c->gexec); c->gexec = nullptr; }
  if (c->graph) { cudaGraphDestroy(c->graph); c->graph = nullptr; }
  const size_t xbytes = (size_t)c->cfg.hidden * c->es;
  CU(cudaStreamSynchronize(c->stream));
  if (n_blocks > MK_MAX_LAYERS) return fail(CAKE_B200_EINVAL, "more than %d blocks per shard", MK_MAX_LAYERS);
  if (n_blocks > 0) {
    std::vector<MkLayer> tab(n_blocks);
    fill_mk_table(tab.data(), blocks, block_idx, n_blocks, kc);
    CU(cudaMemcpy(c->g_tab_dev, tab.data(), sizeof(MkLayer) * n_blocks, cudaMemcpyHostToDevice));
  }
  CU(cudaStreamBeginCapture(c->stream, cudaStreamCaptureModeThreadLocal));
  c->capturing = true;
  c->g_kernels = 0;
  int rc = [&]() -> int {
    if (c->use_mega && mega_supported(c)) {
      // rank 0: [embed+layers(+head if alone)] ; world>1: layers -> send ... recv -> head.  ranks>0: recv -> layers -> send
      MkPlan p;
      const bool p2p = world > 1 && c->inbox && c->peer_inbox;  // hand-off fused into the kernels (no NCCL node)
      unsigned long long *inbox_ctr = (unsigned long long *)c->inbox, *peer_ctr = (unsigned long long *)c->peer_inbox;
      void *inbox_x = c->inbox ? c->inbox + INBOX_X_OFF : nullptr, *peer_x = c->peer_inbox ? c->peer_inbox + INBOX_X_OFF : nullptr;
      if (rank == 0) {
        RC(plan_mega(c, kc, world == 1, &p));
        p.a.layers = c->g_tab_dev; p.a.n_layers = n_blocks; p.a.x_in = nullptr; p.a.x_out = c->xa;
        if (c->cfg.embed_scale != 0.f) {  // text_model.rs:274-276: the scaled embedding row is materialised first
          RC(DISPATCH_T(c->cfg.dtype, T_LAMBDA {
            typedef typename decltype(tag_)::type T;
            return launch_pdl(c, embed_kernel<T>, dim3(1), dim3(128), 0, (const T *)c->embed, (const uint32_t *)c->d_token,
                              (T *)c->x0, 1, c->cfg.hidden, c->cfg.vocab, c->cfg.embed_scale);
          }));
          p.a.x_in = c->x0;
        }
        p.a.has_head = (world == 1); p.a.advance = (world == 1); p.a.token_ring = c->token_ring;
        if (p2p) { p.a.x_out = peer_x; p.a.peer_ctr = peer_ctr; p.a.ring_seq = c->ring_seq; }
        if (n_blocks > 0 || world == 1) RC(launch_mega(c, p));
        if (world > 1) {
          if (n_blocks == 0) return fail(CAKE_B200_EINVAL, "rank 0 must own at least one layer");
          if (!p2p) {
            RC(cake_b200_send(c, c->xa, xbytes, 1));
            RC(cake_b200_recv(c, c->xa, xbytes, world - 1));
          }
          MkPlan h;
          RC(plan_mega(c, kc, true, &h));
          h.a.layers = c->g_tab_dev; h.a.n_layers = 0; h.a.x_in = p2p ? inbox_x : c->xa; h.a.x_out = c->xa;
          h.a.has_head = 1; h.a.advance = 1; h.a.token_ring = c->token_ring; h.a.trace_tag = 1;
          if (p2p) { h.a.inbox_ctr = inbox_ctr; h.a.ring_seq = c->ring_seq; }
          RC(launch_mega(c, h));
        }
        if (c->sampling.kind != SAMPLE_ARGMAX && c->sampling.temperature > 0.f) {
          // non-greedy: a sampler kernel behind the decode kernel re-draws the token from the logits it left behind
          // (256 KB, L2-hot) and overwrites d_token / the ring slot of this step; the step counter was already advanced
          RC(DISPATCH_T(c->cfg.dtype, T_LAMBDA {
            typedef typename decltype(tag_)::type T;
            return launch_pdl(c, sample_kernel<T>, dim3(1), dim3(SAMPLE_THREADS), 0, (const T *)c->logits, c->cfg.vocab, to_args(c->sampling),
                              c->samp_p, (const float *)nullptr, (const int *)c->d_step, -1, c->d_token, c->token_ring, (int)TOKEN_RING);
          }));
        }
      } else {
        if (!p2p) RC(cake_b200_recv(c, c->xa, xbytes, rank - 1));
        RC(plan_mega(c, kc, false, &p));
        p.a.layers = c->g_tab_dev; p.a.n_layers = n_blocks; p.a.x_in = p2p ? inbox_x : c->xa; p.a.x_out = p2p ? peer_x : c->xa;
        p.a.has_head = 0; p.a.advance = 1;
        if (p2p) { p.a.inbox_ctr = inbox_ctr; p.a.peer_ctr = peer_ctr; p.a.ring_seq = c->ring_seq; }
        if (n_blocks > 0) RC(launch_mega(c, p));
        else return fail(CAKE_B200_EINVAL, "every rank must own at least one layer");
        if (!p2p) RC(cake_b200_send(c, c->xa, xbytes, (rank + 1) % world));
      }
      return CAKE_B200_OK;
    }
    if (rank == 0) {
      RC(DISPATCH_T(c->cfg.dtype, T_LAMBDA {
      typedef typename decltype(tag_)::type T;
        return launch_pdl(c, embed_kernel<T>, dim3(1), dim3(128), 0, (const T *)c->embed, (const uint32_t *)c->d_token,
                          (T *)c->xa, 1, c->cfg.hidden, c->cfg.vocab, c->cfg.embed_scale);
      }));
    } else {
      RC(cake_b200_recv(c, c->xa, xbytes, rank - 1));
    }
    if (n_blocks > 0) RC(enqueue_decode_layers(c, blocks, block_idx, n_blocks, kc, c->xa, c->xa));
    if (world > 1) {
      RC(cake_b200_send(c, c->xa, xbytes, (rank + 1) % world));
      if (rank == 0) RC(cake_b200_recv(c, c->xa, xbytes, world - 1));
    }
    if (rank == 0) RC(enqueue_head(c, c->xa, c->logits, true));
    RC(launch_pdl(c, advance_kernel, dim3(1), dim3(32), 0, kc->d_pos, c->d_step));
    return CAKE_B200_OK;
  }();
  c->capturing = false;
  cudaGraph_t g = nullptr;
  cudaError_t e = cudaStreamEndCapture(c->stream, &g);
  if (rc != CAKE_B200_OK) {
    if (g) cudaGraphDestroy(g);
    return rc;
  }
  if (e != cudaSuccess) return fail(CAKE_B200_ECUDA, "graph capture failed: %s", cudaGetErrorString(e));
  c->graph = g;
  CU(cudaGraphInstantiate(&c->gexec, g, 0));
  c->g_cache = kc;
  c->g_block_idx.assign(block_idx, block_idx + n_blocks);
  c->g_rank = rank;
  c->g_world = world;
  return CAKE_B200_OK;
}

extern "C" int cake_b200_decode_begin(cake_b200_ctx *c, uint32_t first_token, int index_pos) {
  if (!c || !c->gexec) return fail(CAKE_B200_ESTATE, "decode_build has not been called");
  CU(cudaSetDevice(c->device));
  RC(wait_loads(c));
  cake_b200_cache *kc = c->g_cache;
  for (int l : c->g_block_idx)
    if (kc->len[l] != index_pos)
      return fail(CAKE_B200_ESTATE, "block %d: index_pos %d != cache length %d", l, index_pos, kc->len[l]);
  if (index_pos >= kc->cap) return fail(CAKE_B200_ESTATE, "cache full");
  if (c->g_rank == 0 && first_token >= (uint32_t)c->cfg.vocab)  // candle's index_select fails on an out-of-range id (text_model.rs:271)
    return fail(CAKE_B200_EINVAL, "token id %u out of range (vocab %d)", first_token, c->cfg.vocab);
  set_int_kernel<<<1, 1, 0, c->stream>>>(kc->d_pos, index_pos);
  set_int_kernel<<<1, 1, 0, c->stream>>>(c->d_step, 0);
  set_u32_kernel<<<1, 1, 0, c->stream>>>(c->d_token, first_token);
  c->launches += 3;
  c->steps_done = 0;
  CU(cudaGetLastError());
  return CAKE_B200_OK;
}

extern "C" int cake_b200_decode_run(cake_b200_ctx *c, int n_steps) {
  if (!c || !c->gexec) return fail(CAKE_B200_ESTATE, "decode_build has not been called");
  CU(cudaSetDevice(c->device));
  cake_b200_cache *kc = c->g_cache;
  int cur = c->g_block_idx.empty() ? 0 : kc->len[c->g_block_idx[0]];
  if (!c->g_block_idx.empty() && cur + n_steps > kc->cap)
    return fail(CAKE_B200_ESTATE, "decode_run: %d steps from position %d exceed cache capacity %d", n_steps, cur, kc->cap);
  for (int i = 0; i < n_steps; i++) CU(cudaGraphLaunch(c->gexec, c->stream));
  for (int l : c->g_block_idx) kc->len[l] += n_steps;
  c->steps_done += n_steps;
  c->launches += c->g_kernels * (uint64_t)n_steps;
  return CAKE_B200_OK;
}

extern "C" int cake_b200_decode_tokens(cake_b200_ctx *c, uint32_t *out_host, int n) {
  if (!c || !out_host || n < 0 || n > TOKEN_RING || n > c->steps_done) return fail(CAKE_B200_EINVAL, "bad decode_tokens arguments");
  CU(cudaSetDevice(c->device));
  CU(cudaStreamSynchronize(c->stream));
  std::vector<uint32_t> ring(TOKEN_RING);
  CU(cudaMemcpy(ring.data(), c->token_ring, (size_t)TOKEN_RING * 4, cudaMemcpyDeviceToHost));
  for (int i = 0; i < n; i++) out_host[i] = ring[(size_t)(c->steps_done - n + i) % TOKEN_RING];
  return CAKE_B200_OK;
}

extern "C" int cake_b200_decode_step_host(cake_b200_ctx *c, uint32_t token_in, uint32_t *token_out) {
  if (!c || !c->gexec || !token_out) return fail(CAKE_B200_ESTATE, "decode_build has not been called");
  CU(cudaSetDevice(c->device));
  if (token_in >= (uint32_t)c->cfg.vocab) return fail(CAKE_B200_EINVAL, "token id %u out of range (vocab %d)", token_in, c->cfg.vocab);
  c->h_pin[32] = token_in;
  CU(cudaMemcpyAsync(c->d_token, c->h_pin + 32, 4, cudaMemcpyHostToDevice, c->stream));
  RC(cake_b200_decode_run(c, 1));
  CU(cudaMemcpyAsync(c->h_pin + 33, c->d_token, 4, cudaMemcpyDeviceToHost, c->stream));
  CU(cudaStreamSynchronize(c->stream));
  *token_out = c->h_pin[33];
  return CAKE_B200_OK;
}

extern "C" int cake_b200_decode_logits(cake_b200_ctx *c, void *logits_host, size_t bytes) {
  if (!c || !logits_host) return fail(CAKE_B200_EINVAL, "null argument");
  const size_t need = (size_t)c->cfg.vocab * c->es;
  if (bytes < need) return fail(CAKE_B200_EINVAL, "decode_logits needs %zu bytes", need);
  CU(cudaSetDevice(c->device));
  CU(cudaStreamSynchronize(c->stream));
  CU(cudaMemcpy(logits_host, c->logits, need, cudaMemcpyDeviceToHost));
  return CAKE_B200_OK;
}

// ------------------------------------------------------------------------------------------ measurement aid
extern "C" int cake_b200_bench_kernel(cake_b200_ctx *c, cake_b200_block *const *blocks, const int *block_idx,
                                      int n_blocks, cake_b200_cache *kc, int which, int reps, float *ms_per_launch) {
  if (!c || !blocks || !kc || !ms_per_launch || n_blocks < 1 || reps < 1 || which < 0 || which > 4)
    return fail(CAKE_B200_EINVAL, "bad bench_kernel arguments");
  for (int i = 0; i < n_blocks; i++)
    if (!blocks[i] || blocks[i]->variant()) return fail(CAKE_B200_EINVAL, "bench_kernel times the per-op kernels of standard blocks only");
  CU(cudaSetDevice(c->device));
  RC(wait_loads(c));
  for (int i = 0; i < n_blocks; i++) RC(cache_ensure(kc, block_idx[i]));
  const int len = kc->len[block_idx[0]];
  if (which == 4 && len < 1) return fail(CAKE_B200_ESTATE, "attention bench needs a non-empty cache");
  if (which == 4) {  // scores the token at position len-1 again: reads len rows, rewrites row len-1
    set_int_kernel<<<1, 1, 0, c->stream>>>(kc->d_pos, len - 1);
  }
  cudaEvent_t e0, e1;
  CU(cudaEventCreate(&e0));
  CU(cudaEventCreate(&e1));
  auto round = [&]() -> int {
    for (int i = 0; i < n_blocks; i++) {
      const cake_b200_block *b = blocks[i];
      switch (which) {
        case 0: RC(enqueue_qkv(c, b, c->xa)); break;
        case 1: RC(enqueue_oproj(c, b, c->xa, c->xb)); break;
        case 2: RC(enqueue_gate_up(c, b, c->xb)); break;
        case 3: RC(enqueue_down(c, b, c->xb, c->xb)); break;
        default: RC(enqueue_attn(c, b, kc, block_idx[i])); break;
      }
    }
    return CAKE_B200_OK;
  };
  RC(round());  // warm-up
  CU(cudaEventRecord(e0, c->stream));
  for (int r = 0; r < reps; r++) RC(round());
  CU(cudaEventRecord(e1, c->stream));
  CU(cudaStreamSynchronize(c->stream));
  float ms = 0.f;
  CU(cudaEventElapsedTime(&ms, e0, e1));
  cudaEventDestroy(e0);
  cudaEventDestroy(e1);
  *ms_per_launch = ms / (float)(reps * n_blocks);
  return CAKE_B200_OK;
}

extern "C" int cake_b200_load_stats(cake_b200_ctx *c, double *bytes, double *seconds) {
  if (!c || !bytes || !seconds) return fail(CAKE_B200_EINVAL, "null argument");
  CU(cudaSetDevice(c->device));
  if (c->load_stream) {  // include the tail of the last DMA in the wall time of the caller, not in `seconds` (host staging time)
    CU(cudaStreamSynchronize(c->load_stream));
  }
  *bytes = c->load_bytes;
  *seconds = c->load_seconds;
  return CAKE_B200_OK;
}

extern "C" int cake_b200_decode_trace(cake_b200_ctx *c, uint64_t *out_host, int n_steps) {
  if (!c || !out_host || n_steps < 0 || n_steps > MK_STEP_RING || n_steps > c->steps_done)
    return fail(CAKE_B200_EINVAL, "bad decode_trace arguments (at most %d of the steps since decode_begin)", MK_STEP_RING);
  CU(cudaSetDevice(c->device));
  CU(cudaStreamSynchronize(c->stream));
  std::vector<unsigned long long> ring((size_t)MK_STEP_RING * 8);
  CU(cudaMemcpy(ring.data(), c->step_trace, ring.size() * 8, cudaMemcpyDeviceToHost));
  for (int i = 0; i < n_steps; i++) {
    const size_t slot = (size_t)((c->steps_done - n_steps + i) % MK_STEP_RING) * 8;
    for (int j = 0; j < 8; j++) out_host[(size_t)i * 8 + j] = ring[slot + j];
  }
  return CAKE_B200_OK;
}

/* profiling aid (not in the public header): copies the megakernel's phase-boundary %globaltimer stamps of
 * the last launch (CTA 0) to `out`; needs CAKE_B200_MEGA_TRACE=1 at ctx creation. */
extern "C" int cake_b200_debug_trace(cake_b200_ctx *c, unsigned long long *out, int n) {
  if (!c || !c->trace || n > 4096) return fail(CAKE_B200_ESTATE, "tracing is off (CAKE_B200_MEGA_TRACE=1)");
  CU(cudaSetDevice(c->device));
  CU(cudaStreamSynchronize(c->stream));
  CU(cudaMemcpy(out, c->trace, (size_t)n * 8, cudaMemcpyDeviceToHost));
  return CAKE_B200_OK;
}
