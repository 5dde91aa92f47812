// Host runtime of the fused AllReduce: context, window geometry, argument validation, shape lookup
// and the launch itself (programmatic dependent launch in production, cooperative launch when several
// ranks are emulated on one device).
//
// Reference project counterparts: kernels/push/tp2_l2.cu:956-1066 (layout / init_impl / launch_impl),
// kernels/fused_norm/lnorm.cu:703-770.  The window here is 2 buffers of max(P*cap, 2*P*ceil(cap/P))
// slots of 3584 B, shared by every algorithm and input kind (the reference keeps 3 buffers for each of
// one-shot, two-shot and NVFP4-input regions).
#include <cstdio>
#include <cstdlib>
#include <atomic>
#include <cstring>
#include <memory>
#include <mutex>
#include <string>
#include <utility>
#include <vector>
#include "../include/fp4ar.h"
#include "../kernels/ar_table.h"
#include "../kernels/host_util.h"

namespace fp4ar {

static std::mutex g_mu;
static std::string g_last_error = "";

void set_last_cuda_error(cudaError_t e, const char* where) {
  std::lock_guard<std::mutex> lk(g_mu);
  g_last_error = std::string(where) + ": " + cudaGetErrorName(e) + " (" + cudaGetErrorString(e) + ")";
}
int cuda_fail() {
  set_last_cuda_error(cudaGetLastError(), "cuda");
  return FP4AR_ERR_CUDA;
}
int cuda_check_launch() {
  const cudaError_t e = cudaGetLastError();
  if (e == cudaSuccess) return FP4AR_OK;
  set_last_cuda_error(e, "launch");
  return FP4AR_ERR_CUDA;
}
int device_sm_count() {
  static std::atomic<int> cache[64];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 1;
  int n = cache[dev].load(std::memory_order_relaxed);
  if (!n) {
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 1;
    cache[dev].store(n, std::memory_order_relaxed);   // every thread computes the same value
  }
  return n;
}

#define FP4AR_CUDA(call)                                    \
  do {                                                      \
    const cudaError_t e_ = (call);                          \
    if (e_ != cudaSuccess) {                                \
      set_last_cuda_error(e_, #call);                       \
      return FP4AR_ERR_CUDA;                                \
    }                                                       \
  } while (0)

static std::vector<ArKernelEntry>& kernel_table() {
  static std::vector<ArKernelEntry> table;
  static std::once_flag once;
  std::call_once(once, [] {
    ArKernelEntry buf[256];
    int n = 0;
    ar_register_p1(buf, &n); ar_register_p2(buf, &n); ar_register_p2b(buf, &n);
    ar_register_p4(buf, &n); ar_register_p4b(buf, &n); ar_register_p8(buf, &n); ar_register_p8b(buf, &n);
    ar_register_cmp(buf, &n);
    ar_register_t6p4(buf, &n); ar_register_t6p4b(buf, &n); ar_register_t6p8(buf, &n); ar_register_t6p8b(buf, &n);
    table.assign(buf, buf + n);
  });
  return table;
}
static const ArKernelEntry* find_kernel(int P, int algo, int input, int epi, int T) {
  for (const ArKernelEntry& e : kernel_table())
    if (e.P == P && e.algo == algo && e.input == input && e.epi == epi && e.T == T) return &e;
  return nullptr;
}
// Team width: tune[2] of the call if set, else FP4AR_TEAM_WARPS from the environment (a preference: shapes that are
// not compiled at that width use their default), else the default of the shape.
static int team_warps_for(const fp4ar_args& a, int nranks, int algo) {
  if (a.tune[2] > 0) return a.tune[2];
  static const int from_env = [] {
    const char* s = std::getenv("FP4AR_TEAM_WARPS");
    const int v = s ? std::atoi(s) : 0;
    return v > 0 ? v : 0;
  }();
  return from_env > 0 ? from_env : default_team_warps(nranks, algo);
}

#ifdef FP4AR_PHASE_TIMERS
}  // namespace fp4ar
static unsigned long long* phase_buffer();
namespace fp4ar {
#endif

struct Geometry {
  int cap, capo;
  size_t buf_bytes, total;
};
static Geometry geometry(int max_rows, int nranks) {
  Geometry g;
  g.cap = max_rows;
  g.capo = (max_rows + nranks - 1) / nranks;
  size_t slots = (size_t)nranks * g.cap;
  const size_t two = 2 * (size_t)nranks * g.capo;
  if (two > slots) slots = two;
  g.buf_bytes = (slots * kRecStride + 4095) / 4096 * 4096;
  g.total = (2 * g.buf_bytes + (2u << 20) - 1) / (2u << 20) * (2u << 20);
  return g;
}

}  // namespace fp4ar

using namespace fp4ar;

struct fp4ar_ctx {
  int rank = 0, nranks = 0, device = 0, max_rows = 0;
  int nlocal = 0;        // ranks run by one launch (1, or nranks when emulated)
  bool emulated = false;
  int ctas_per_rank = 0;
  Geometry geo{};
  size_t window_bytes = 0;
  char* win[FP4AR_MAX_RANKS] = {};
  uint32_t* ctrl[FP4AR_MAX_RANKS] = {};
  StatusWords* status[FP4AR_MAX_RANKS] = {};
  // One word of pinned, device-mapped host memory: a wait that gives up stores its status code here, and
  // fp4ar_launch reads it on the host (no synchronisation) to refuse further calls until fp4ar_reset.
  uint32_t* poison_host = nullptr;
  uint32_t* poison_dev = nullptr;
  unsigned long long timeout_ns = 0;
  int max_smem_optin = 0;
  // kernels whose dynamic shared-memory limit this context has already raised (function, bytes)
  std::vector<std::pair<const void*, int>> smem_raised;
  std::mutex mu;

  ~fp4ar_ctx() {
    for (int l = 0; l < FP4AR_MAX_RANKS; l++) {
      if (ctrl[l]) cudaFree(ctrl[l]);
      if (status[l]) cudaFree(status[l]);
    }
    if (poison_host) cudaFreeHost(poison_host);
  }
};

extern "C" size_t fp4ar_window_bytes(int max_rows, int hidden, int nranks) {
  if (hidden != FP4AR_HIDDEN || max_rows < 1 || nranks < 1 || nranks > FP4AR_MAX_RANKS) return 0;
  if (nranks != 1 && nranks != 2 && nranks != 4 && nranks != 8) return 0;
  return geometry(max_rows, nranks).total;
}

static int create_common(fp4ar_ctx** out, int rank, int nranks, int device, int max_rows, int hidden,
                         void* const* windows, size_t window_bytes, bool emulated) {
  if (!out || !windows) return FP4AR_ERR_ARGUMENT;
  const size_t need = fp4ar_window_bytes(max_rows, hidden, nranks);
  if (need == 0 || window_bytes < need) return FP4AR_ERR_ARGUMENT;
  if (!emulated && (rank < 0 || rank >= nranks)) return FP4AR_ERR_ARGUMENT;
  for (int r = 0; r < nranks; r++)
    if (!windows[r] || ((uintptr_t)windows[r] & 255)) return FP4AR_ERR_ARGUMENT;
  FP4AR_CUDA(cudaSetDevice(device));
  std::unique_ptr<fp4ar_ctx> c(new fp4ar_ctx());   // freed, with its device buffers, on every error return below
  c->rank = rank; c->nranks = nranks; c->device = device; c->max_rows = max_rows;
  c->emulated = emulated; c->nlocal = emulated ? nranks : 1;
  c->geo = geometry(max_rows, nranks);
  c->window_bytes = window_bytes;
  {
    // how long a device-side wait may last: 10 s unless FP4AR_TIMEOUT_MS or fp4ar_set_timeout_ms says otherwise
    const char* e = std::getenv("FP4AR_TIMEOUT_MS");
    const long ms = e ? std::atol(e) : 0;
    c->timeout_ns = (unsigned long long)(ms > 0 ? ms : 10000) * 1000000ull;
  }
  for (int r = 0; r < nranks; r++) c->win[r] = (char*)windows[r];
  int sms = 0;
  FP4AR_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device));
  FP4AR_CUDA(cudaDeviceGetAttribute(&c->max_smem_optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, device));
  c->ctas_per_rank = emulated ? sms / nranks : sms;
  if (c->ctas_per_rank < 1) return FP4AR_ERR_UNSUPPORTED;
  FP4AR_CUDA(cudaHostAlloc((void**)&c->poison_host, 64, cudaHostAllocMapped));
  *c->poison_host = 0u;
  FP4AR_CUDA(cudaHostGetDevicePointer((void**)&c->poison_dev, c->poison_host, 0));
  for (int l = 0; l < c->nlocal; l++) {
    FP4AR_CUDA(cudaMalloc(&c->ctrl[l], sizeof(uint32_t) * c->ctas_per_rank));
    FP4AR_CUDA(cudaMemset(c->ctrl[l], 0, sizeof(uint32_t) * c->ctas_per_rank));
    FP4AR_CUDA(cudaMalloc(&c->status[l], sizeof(StatusWords)));
    FP4AR_CUDA(cudaMemset(c->status[l], 0, sizeof(StatusWords)));
  }
  // arm the local window(s)
  for (int l = 0; l < c->nlocal; l++) {
    char* w = emulated ? c->win[l] : c->win[rank];
    const int rc = fp4ar_fill_sentinel(w, c->geo.buf_bytes, 2, nullptr);
    if (rc != FP4AR_OK) return rc;
  }
  FP4AR_CUDA(cudaDeviceSynchronize());
  *out = c.release();
  return FP4AR_OK;
}

extern "C" int fp4ar_create(fp4ar_ctx** ctx, int rank, int nranks, int device, int max_rows, int hidden,
                            void* const* windows, size_t window_bytes) {
  return create_common(ctx, rank, nranks, device, max_rows, hidden, windows, window_bytes, false);
}
extern "C" int fp4ar_create_emulated(fp4ar_ctx** ctx, int nranks, int device, int max_rows, int hidden,
                                     void* const* windows, size_t window_bytes) {
  return create_common(ctx, 0, nranks, device, max_rows, hidden, windows, window_bytes, true);
}

extern "C" int fp4ar_destroy(fp4ar_ctx* c) {
  if (!c) return FP4AR_ERR_ARGUMENT;
  delete c;
  return FP4AR_OK;
}

extern "C" int fp4ar_set_timeout_ms(fp4ar_ctx* c, int ms) {
  if (!c || ms < 1) return FP4AR_ERR_ARGUMENT;
  c->timeout_ns = (unsigned long long)ms * 1000000ull;
  return FP4AR_OK;
}

extern "C" int fp4ar_status(fp4ar_ctx* c, int local_rank, fp4ar_status_words* out) {
  if (!c || !out || local_rank < 0 || local_rank >= c->nlocal) return FP4AR_ERR_ARGUMENT;
  static_assert(sizeof(fp4ar_status_words) == sizeof(StatusWords), "status layout");
  FP4AR_CUDA(cudaMemcpy(out, c->status[local_rank], sizeof(StatusWords), cudaMemcpyDeviceToHost));
  return FP4AR_OK;
}

extern "C" int fp4ar_reset(fp4ar_ctx* c) {
  if (!c) return FP4AR_ERR_ARGUMENT;
  FP4AR_CUDA(cudaDeviceSynchronize());
  for (int l = 0; l < c->nlocal; l++) {
    char* w = c->emulated ? c->win[l] : c->win[c->rank];
    const int rc = fp4ar_fill_sentinel(w, c->geo.buf_bytes, 2, nullptr);
    if (rc != FP4AR_OK) return rc;
    FP4AR_CUDA(cudaMemset(c->status[l], 0, sizeof(StatusWords)));
    FP4AR_CUDA(cudaMemset(c->ctrl[l], 0, sizeof(uint32_t) * c->ctas_per_rank));
  }
  FP4AR_CUDA(cudaDeviceSynchronize());
  *reinterpret_cast<volatile uint32_t*>(c->poison_host) = 0u;
  return FP4AR_OK;
}

extern "C" int fp4ar_ctas_per_rank(fp4ar_ctx* c) { return c ? c->ctas_per_rank : 0; }

extern "C" int fp4ar_get_push_view(fp4ar_ctx* c, int local_rank, fp4ar_push_view* out) {
  if (!c || !out || local_rank < 0 || local_rank >= c->nlocal) return FP4AR_ERR_ARGUMENT;
  out->call_counter = c->ctrl[local_rank];
  out->buffer_bytes = c->geo.buf_bytes;
  out->cap = c->geo.cap; out->capo = c->geo.capo;
  out->nranks = c->nranks; out->rank = c->emulated ? local_rank : c->rank;
  for (int r = 0; r < FP4AR_MAX_RANKS; r++) out->windows[r] = r < c->nranks ? c->win[r] : nullptr;
  return FP4AR_OK;
}

extern "C" const char* fp4ar_last_cuda_error(void) {
  std::lock_guard<std::mutex> lk(g_mu);
  static thread_local std::string copy;
  copy = g_last_error;
  return copy.c_str();
}

extern "C" int fp4ar_has_kernel(int nranks, int algo, int input, int epilogue, int team_warps) {
  const ArKernelEntry* e = find_kernel(nranks, algo, input, epilogue, team_warps);
  return e && e->fn ? e->max_teams : 0;
}
extern "C" int fp4ar_default_team_warps(int nranks, int algo) { return default_team_warps(nranks, algo); }

extern "C" const char* fp4ar_build_info(void) {
  static std::string s;
  if (s.empty()) {
    char b[256];
    std::snprintf(b, sizeof(b), "fp4ar sm_100a cuda-runtime %d shapes %d team-warps %d", CUDART_VERSION,
                  (int)kernel_table().size(), kDefaultTeamWarps);
    s = b;
  }
  return s.c_str();
}

static bool aligned16(const void* p) { return ((uintptr_t)p & 15) == 0; }

extern "C" int fp4ar_launch(fp4ar_ctx* c, const fp4ar_args* args, fp4ar_stream stream) {
  if (!c || !args) return FP4AR_ERR_ARGUMENT;
  const fp4ar_args& a0 = args[0];
  if (a0.hidden != FP4AR_HIDDEN || a0.rows < 0 || a0.rows > c->max_rows) return FP4AR_ERR_ARGUMENT;
  if (a0.mode < 0 || a0.mode > 2 || a0.input < 0 || a0.input > 2 || a0.epilogue < 0 || a0.epilogue > 3)
    return FP4AR_ERR_ARGUMENT;
  // A wait of an earlier call gave up: some receive slots may still hold data or miss their re-arm, so every
  // later result would be wrong.  The word is written by the device into mapped host memory; reading it costs
  // no synchronisation (a call enqueued before the failing kernel ran cannot see it yet).
  if (*reinterpret_cast<volatile uint32_t*>(c->poison_host) != 0u) return FP4AR_ERR_POISONED;
  // Nothing to reduce: no launch, so the device call counter (and with it the buffer parity) does not move.
  if (a0.rows == 0) return FP4AR_OK;
  int algo = a0.algo;
  if (algo == FP4AR_ALGO_AUTO) algo = c->nranks <= 2 ? FP4AR_ALGO_ONESHOT : FP4AR_ALGO_TWOSHOT;
  if (algo != FP4AR_ALGO_ONESHOT && algo != FP4AR_ALGO_TWOSHOT) return FP4AR_ERR_ARGUMENT;
  if (c->nranks == 1) algo = FP4AR_ALGO_ONESHOT;
  const ArKernelEntry* ke = find_kernel(c->nranks, algo, a0.input, a0.epilogue, team_warps_for(a0, c->nranks, algo));
  // a team width that comes from the environment is a preference: shapes not compiled at that width use their default
  if (!ke && a0.tune[2] <= 0) ke = find_kernel(c->nranks, algo, a0.input, a0.epilogue, default_team_warps(c->nranks, algo));
  if (!ke) return FP4AR_ERR_UNSUPPORTED;

  ArParams prm;
  std::memset(&prm, 0, sizeof(prm));
  for (int l = 0; l < c->nlocal; l++) {
    const fp4ar_args& a = args[l];
    // every local rank must describe the same call
    if (a.rows != a0.rows || a.hidden != a0.hidden || a.mode != a0.mode || a.algo != a0.algo || a.input != a0.input ||
        a.epilogue != a0.epilogue)
      return FP4AR_ERR_ARGUMENT;
    if (a.input != FP4AR_IN_PUSHED && (!a.x || !aligned16(a.x))) return FP4AR_ERR_ARGUMENT;
    if (a.epilogue <= FP4AR_EPI_NORM_BF16 && (!a.out || !aligned16(a.out))) return FP4AR_ERR_ARGUMENT;
    if (a.epilogue != FP4AR_EPI_NONE) {
      if (!a.res_in || !a.res_out || !a.weight || !aligned16(a.res_in) || !aligned16(a.res_out) || !aligned16(a.weight))
        return FP4AR_ERR_ARGUMENT;
      if (a.weight != a0.weight || a.eps != a0.eps || a.weight_bias != a0.weight_bias || a.qscale != a0.qscale)
        return FP4AR_ERR_ARGUMENT;
      if (a.epilogue >= FP4AR_EPI_NORM_NVFP4 && (!a.outq || !aligned16(a.outq))) return FP4AR_ERR_ARGUMENT;
    }
    if (a.input != FP4AR_IN_BF16)
      for (int r = 0; r < c->nranks; r++)
        if (!(a.gs[r] > 0.0f) || a.gs[r] != a0.gs[r]) return FP4AR_ERR_ARGUMENT;
    RankIO& io = prm.io[l];
    io.x = (const char*)a.x; io.out = (char*)a.out;
    io.res_in = (const char*)a.res_in; io.res_out = (char*)a.res_out; io.outq = (char*)a.outq;
    for (int r = 0; r < c->nranks; r++) io.win[r] = c->win[r];
    io.ctrl = c->ctrl[l]; io.status = c->status[l]; io.poison = c->poison_dev;
    io.rank = c->emulated ? l : c->rank;
  }
  prm.weight = (const char*)a0.weight;
  for (int r = 0; r < FP4AR_MAX_RANKS; r++) prm.gs[r] = a0.gs[r];
  prm.eps = a0.eps; prm.wbias = a0.weight_bias; prm.qscale = a0.qscale;
  prm.rows = a0.rows; prm.ctas_per_rank = c->ctas_per_rank;
  prm.flags = (a0.mode == FP4AR_MODE_XPORT ? kFlagXport : 0) | (a0.mode == FP4AR_MODE_COMPUTE ? kFlagLoopback : 0);
  prm.cap = c->geo.cap; prm.capo = c->geo.capo;
  prm.buf_bytes = c->geo.buf_bytes; prm.timeout_ns = c->timeout_ns;
  // Two-shot pipeline depths: tune[3] = lag_owner | lag_finish << 4 when set, otherwise by team width and degree.
  // Three-warp teams (measured on 4 and 8 GPUs): (1,2) at four ranks, where the kernel is bound by its own codec work
  // at large row counts and the shallow pipeline wins; (2,3) at eight, where every row waits on seven peers and one
  // more step of slack at each hand-off pays at every row count (16K rows: 284 -> 228 us).  A step of a six-warp team
  // takes about half as long, so those shapes run (2,3) everywhere.  Eight GPUs, 16384 rows, AR / block: (2,3) 179 /
  // 238 us, (2,4) 192 / 240, (3,4) 181 / 240; 1024 rows: 24.6, 27.6, 23.2 us.  Four GPUs, 16384 rows: (1,2) 209 / 231,
  // (2,3) 150 / 199, (2,4) 156 / 202, (3,4) 154 / 201; 1024 rows: 23.6, 17.8, 18.8, 18.6 us.
  {
    int lo = a0.tune[3] & 15, lf = (a0.tune[3] >> 4) & 15;
    if (lo < 1 || lf <= lo || lf > 4) {
      if (ke->T == 6 || c->nranks >= 6) { lo = 2; lf = 3; }
      else { lo = 1; lf = 2; }
    }
    prm.lag_owner = lo; prm.lag_finish = lf;
  }
#ifdef FP4AR_PHASE_TIMERS
  prm.phase_cycles = phase_buffer();
#endif

  // host-side bounds check of the largest window offset this call can touch
  {
    const size_t last_os = ((size_t)(c->nranks - 1) * prm.cap + (size_t)(a0.rows > 0 ? a0.rows - 1 : 0)) * kRecStride;
    const size_t last_ts = ((size_t)(2 * c->nranks - 1) * prm.capo + (size_t)(a0.rows > 0 ? (a0.rows - 1) / c->nranks : 0)) * kRecStride;
    const size_t last = (algo == FP4AR_ALGO_ONESHOT ? last_os : last_ts) + kRecStride;
    if (last > c->geo.buf_bytes || 2 * c->geo.buf_bytes > c->window_bytes) return FP4AR_ERR_ARGUMENT;
  }

  int teams = ke->max_teams;
  const int fit = (c->max_smem_optin - ke->cta_extra) / ke->team_bytes;
  if (fit < teams) teams = fit;
  if (a0.tune[0] > 0 && a0.tune[0] < teams) teams = a0.tune[0];
  if (teams < 1) return FP4AR_ERR_UNSUPPORTED;
  const int smem = teams * ke->team_bytes + ke->cta_extra;
  {
    // the limit is raised once per (context, kernel), not on every launch
    std::lock_guard<std::mutex> lk(c->mu);
    bool done = false;
    for (auto& e : c->smem_raised)
      if (e.first == ke->fn) {
        if (e.second >= smem) done = true;
        else { FP4AR_CUDA(cudaFuncSetAttribute(ke->fn, cudaFuncAttributeMaxDynamicSharedMemorySize, smem)); e.second = smem; done = true; }
        break;
      }
    if (!done) {
      FP4AR_CUDA(cudaFuncSetAttribute(ke->fn, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
      c->smem_raised.emplace_back(ke->fn, smem);
    }
  }

  cudaLaunchConfig_t cfg;
  std::memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = dim3((unsigned)(c->ctas_per_rank * c->nlocal), 1, 1);
  cfg.blockDim = dim3((unsigned)(teams * ke->T * 32), 1, 1);
  cfg.dynamicSmemBytes = (size_t)smem;
  cfg.stream = (cudaStream_t)stream;
  cudaLaunchAttribute attr[1];
  if (c->emulated) {
    attr[0].id = cudaLaunchAttributeCooperative;
    attr[0].val.cooperative = 1;
    cfg.attrs = attr; cfg.numAttrs = 1;
  } else if (!(a0.tune[1] & 1)) {
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr; cfg.numAttrs = 1;
  }
  void* kargs[1] = {&prm};
  FP4AR_CUDA(cudaLaunchKernelExC(&cfg, ke->fn, kargs));
  return FP4AR_OK;
}

#ifdef FP4AR_PHASE_TIMERS
// Tuning builds only: per-phase cycle counters filled by the kernel (see FP4AR_PHASE in ar_kernel.cuh).
static unsigned long long* g_phase_dev = nullptr;
static unsigned long long* phase_buffer() {
  if (!g_phase_dev) { cudaMalloc(&g_phase_dev, 16 * sizeof(unsigned long long)); cudaMemset(g_phase_dev, 0, 16 * sizeof(unsigned long long)); }
  return g_phase_dev;
}
extern "C" int fp4ar_debug_phase_cycles(unsigned long long* out16) {
  if (cudaMemcpy(out16, phase_buffer(), 16 * sizeof(unsigned long long), cudaMemcpyDeviceToHost) != cudaSuccess) return FP4AR_ERR_CUDA;
  cudaMemset(phase_buffer(), 0, 16 * sizeof(unsigned long long));
  return FP4AR_OK;
}
#endif
