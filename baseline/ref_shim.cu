// Driver for the UNMODIFIED kernels of the reference project (fans-nv/fp4-all-reduce) on this machine.
//
// The reference's own harness (harness/fp4ar_bench.cu) obtains peer pointers from NCCL >= 2.31
// (ncclGetLsaDevicePointer), which the NCCL on this image (2.28.9) does not have.  This driver supplies the same
// `Fp4ArCtx` the reference's variants expect -- rank, nranks, sm_count, an NCCL communicator (the variants use it
// for one 1-float all-reduce at init) and peer[] -- from plain CUDA peer access: one host thread per GPU in one
// process (as in the reference harness), windows from cudaMalloc, cudaDeviceEnablePeerAccess between all pairs.
// Everything on the device is the reference's code, compiled from an untouched copy of its sources and called
// through its own variant interface (include/fp4ar_api.h: window_bytes / init / launch / fini, and the
// lnorm_* functions of kernels/fused_norm/lnorm.cu).
//
// Timing protocol = the reference's (harness/fp4ar_bench.cu:154-187): a CUDA graph of K calls, ranks aligned by a
// host barrier and a 1-element all-reduce before every iteration, CUDA events around the replay, per-iteration
// maximum over ranks, median over iterations.  Prints one JSON line.
//
//   ref_shim --tp 2 --variant L2|L4|lnorm --rows 16384 [--input bf16|nvfp4] [--epi 0..3] [--algo 0|1]
//            [--graph 10] [--iters 50] [--warmup 10] [--in prefix] [--dump prefix]
//            [--nsets 1] [--mode 0|1|2] [--solo 0|1] [--e2e 0|1]
// --nsets n    : the K calls of the graph read n rotating copies of the input (copy i = the rows rolled by i), so that
//                with n x rows x 12 KB > 2 x L2 no call finds its input in the cache
// --mode       : the reference's Fp4ArMode (0 fused, 1 transport only, 2 compute only: same codec work, no peer traffic)
// --solo 1     : run rank 0 of a --tp group ALONE on GPU 0 (needs --mode 2, where the kernel neither pushes nor waits)
// --e2e 1      : additionally time, per iteration, pinned host -> device copies of one input set and of the residual, the
//                graph, and a 32-byte device -> host read of the result, in one event-bracketed region
// --in  prefix : read rank r's BF16 input from <prefix>.x<r>.bin (and <prefix>.res.bin, <prefix>.w.bin for lnorm)
// --dump prefix: write rank 0's BF16 output of the first call to <prefix>.out.bin (and .res_out.bin)
#include <algorithm>
#include <atomic>
#include <condition_variable>
#include <cstdio>
#include <cstdlib>
#include <cmath>
#include <cstring>
#include <mutex>
#include <random>
#include <string>
#include <thread>
#include <unistd.h>
#include <vector>
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <nccl.h>
#include "fp4ar_api.h"
#include "lnorm_epi.cuh"
#include "ref.cuh"   // the reference harness' own input quantiser (ref::q_encode) for --input nvfp4

const Fp4ArVariant* fp4ar_register_L2();
const Fp4ArVariant* fp4ar_register_L4();
size_t lnorm_window_bytes(int max_rows, int hidden, int nranks);
int lnorm_init(Fp4ArCtx* c, int max_rows, int hidden);
int lnorm_launch(Fp4ArCtx* c, const Fp4ArArgs* a, const lne::NormArgs* n, cudaStream_t s);
void lnorm_fini(Fp4ArCtx* c);

#define CK(x) do { cudaError_t e_ = (x); if (e_ != cudaSuccess) { fprintf(stderr, "CUDA %s at %s:%d\n", cudaGetErrorString(e_), __FILE__, __LINE__); _exit(5); } } while (0)
#define NK(x) do { ncclResult_t e_ = (x); if (e_ != ncclSuccess) { fprintf(stderr, "NCCL %s at %s:%d\n", ncclGetErrorString(e_), __FILE__, __LINE__); _exit(6); } } while (0)

struct HostBarrier {
  std::mutex m; std::condition_variable cv; int n, count = 0, gen = 0;
  explicit HostBarrier(int n_) : n(n_) {}
  void wait() { std::unique_lock<std::mutex> l(m); int g = gen; if (++count == n) { count = 0; gen++; cv.notify_all(); } else cv.wait(l, [&] { return g != gen; }); }
};

struct Opts {
  int tp = 2, rows = 16384, epi = 0, algo = -1, graph = 10, iters = 50, warmup = 10;
  int nsets = 1, mode = 0, solo = 0, e2e = 0;
  std::string variant = "L2", input = "bf16", in, dump;
};
static Opts g;
static std::vector<std::vector<float>> g_times;   // [rank][iter] ms
static std::vector<std::vector<float>> g_e2e;     // [rank][iter] ms, --e2e 1
static size_t g_h2d = 0, g_d2h = 0;
static float g_gs[8] = {1, 1, 1, 1, 1, 1, 1, 1};   // --input nvfp4: static scale of every rank's partial (amax / 2688)
static constexpr int H = 6144;

static std::vector<uint16_t> read_file(const std::string& p, size_t n) {
  std::vector<uint16_t> v(n);
  FILE* f = fopen(p.c_str(), "rb");
  if (!f || fread(v.data(), 2, n, f) != n) { fprintf(stderr, "cannot read %s\n", p.c_str()); _exit(7); }
  fclose(f);
  return v;
}
static void write_file(const std::string& p, const void* d, size_t bytes) {
  FILE* f = fopen(p.c_str(), "wb");
  if (!f || fwrite(d, 1, bytes, f) != bytes) { fprintf(stderr, "cannot write %s\n", p.c_str()); _exit(7); }
  fclose(f);
}
static uint16_t f2bf(float f) { uint32_t u; memcpy(&u, &f, 4); u += 0x7fff + ((u >> 16) & 1); return (uint16_t)(u >> 16); }

static void worker(int rank, ncclUniqueId id, HostBarrier* bar, std::vector<char*>* windows, size_t win_bytes) {
  CK(cudaSetDevice(rank));
  const int nthreads = g.solo ? 1 : g.tp;
  if (!g.solo)
    for (int r = 0; r < g.tp; r++) if (r != rank) { cudaError_t e = cudaDeviceEnablePeerAccess(r, 0); if (e != cudaSuccess && e != cudaErrorPeerAccessAlreadyEnabled) CK(e); cudaGetLastError(); }
  ncclComm_t comm; NK(ncclCommInitRank(&comm, nthreads, id, rank));
  cudaStream_t st; CK(cudaStreamCreate(&st));
  const size_t n = (size_t)g.rows * H;
  // inputs
  std::vector<uint16_t> hx(n), hres, hw;
  if (!g.in.empty()) hx = read_file(g.in + ".x" + std::to_string(rank) + ".bin", n);
  else { std::mt19937 rng(1234 + rank); std::normal_distribution<float> nd(0.f, 1.f); std::vector<uint16_t> blk(1 << 20); for (auto& v : blk) v = f2bf(nd(rng)); for (size_t i = 0; i < n; i++) hx[i] = blk[(i * 2654435761u) & ((1 << 20) - 1)]; }
  __nv_bfloat16 *x, *out, *res = nullptr, *w = nullptr; float* one;
  CK(cudaMalloc(&x, n * 2)); CK(cudaMalloc(&out, n * 2)); CK(cudaMalloc(&one, 4)); CK(cudaMemset(one, 0, 4));
  CK(cudaMemcpy(x, hx.data(), n * 2, cudaMemcpyHostToDevice));
  // rotating input sets: set i = the rows of x rolled by i
  std::vector<__nv_bfloat16*> xset(1, x);
  for (int i = 1; i < g.nsets; i++) {
    __nv_bfloat16* xi; CK(cudaMalloc(&xi, n * 2));
    const size_t head = (size_t)(i % g.rows) * H;
    CK(cudaMemcpy(xi + head, x, (n - head) * 2, cudaMemcpyDeviceToDevice));
    if (head) CK(cudaMemcpy(xi, x + (n - head), head * 2, cudaMemcpyDeviceToDevice));
    xset.push_back(xi);
  }
  const bool norm = g.variant == "lnorm";
  if (norm) {
    if (!g.in.empty()) { hres = read_file(g.in + ".res.bin", n); hw = read_file(g.in + ".w.bin", H); }
    else { hres.assign(hx.begin(), hx.end()); hw.assign(H, f2bf(0.01f)); }
    CK(cudaMalloc(&res, n * 2)); CK(cudaMalloc(&w, H * 2));
    CK(cudaMemcpy(res, hres.data(), n * 2, cudaMemcpyHostToDevice)); CK(cudaMemcpy(w, hw.data(), H * 2, cudaMemcpyHostToDevice));
  }
  // window
  char* win; CK(cudaMalloc(&win, win_bytes)); CK(cudaMemset(win, 0, win_bytes));
  (*windows)[rank] = win;
  CK(cudaDeviceSynchronize());
  bar->wait();
  Fp4ArCtx ctx{}; ctx.rank = rank; ctx.nranks = g.tp; ctx.device = rank; ctx.comm = comm; ctx.win_bytes = win_bytes;
  cudaDeviceProp prop; CK(cudaGetDeviceProperties(&prop, rank)); ctx.sm_count = prop.multiProcessorCount;
  for (int r = 0; r < g.tp; r++) ctx.peer[r] = g.solo ? win : (*windows)[r];   // alone: every "peer" is this window (compute mode never pushes)
  const Fp4ArVariant* V = g.variant == "L2" ? fp4ar_register_L2() : g.variant == "L4" ? fp4ar_register_L4() : nullptr;
  int rc = norm ? lnorm_init(&ctx, g.rows, H) : V->init(&ctx, g.rows, H);
  if (rc) { fprintf(stderr, "variant init failed on rank %d\n", rank); _exit(8); }
  Fp4ArArgs a{}; a.x = x; a.out = out; a.rows = g.rows; a.hidden = H; a.mode = g.mode;
  a.algo = g.algo >= 0 ? g.algo : (g.tp == 2 ? FP4AR_ONESHOT : (norm ? FP4AR_ONESHOT : FP4AR_TWOSHOT));
  for (int r = 0; r < 8; r++) a.gs[r] = 1.0f;
  std::vector<const uint8_t*> xqset;
  if (g.input == "nvfp4") {
    // The way the reference harness emulates calibration (harness/fp4ar_bench.cu:206-215): gs = amax of the rank's
    // partial / 2688, known to every rank; the partial is quantised once, outside the timed region, by the
    // reference's own ref::q_encode, and the kernels read the 3456-byte rows from a local buffer.
    float am = 0.f;
    for (size_t i = 0; i < n; i++) { uint32_t u = (uint32_t)hx[i] << 16; float f; memcpy(&f, &u, 4); f = fabsf(f); if (f == f && f > am) am = f; }
    g_gs[rank] = (am > 0.f ? am : 1.f) / 2688.f;
    bar->wait();
    for (int r = 0; r < g.tp; r++) a.gs[r] = g_gs[r];
    for (int i = 0; i < g.nsets; i++) {
      char* xq; CK(cudaMalloc(&xq, (size_t)g.rows * 3456));
      ref::q_encode<<<2048, 256, 0, st>>>(xset[i], xq, g.rows, g_gs[rank]);
      xqset.push_back((const uint8_t*)xq);
    }
    CK(cudaStreamSynchronize(st));
    a.xq = xqset[0]; a.xq_in_window = 0;
    if (rank == 0 && !g.dump.empty()) write_file(g.dump + ".gs.bin", g_gs, sizeof(float) * g.tp);
  }
  lne::NormArgs na{}; na.res_in = res; na.res_out = res; na.w = w; na.eps = 1e-6f; na.wbias = 1.0f; na.epi = g.epi; na.outq = nullptr; na.qscale = 168.0f;
  auto op_set = [&](int i) { a.x = xset[i % g.nsets]; if (!xqset.empty()) a.xq = xqset[i % g.nsets]; };
  auto op = [&]() { int r2 = norm ? lnorm_launch(&ctx, &a, &na, st) : V->launch(&ctx, &a, st); if (r2) { fprintf(stderr, "launch rejected on rank %d\n", rank); _exit(9); } };
  auto align = [&]() { CK(cudaStreamSynchronize(st)); bar->wait(); NK(ncclAllReduce(one, one, 1, ncclFloat, ncclSum, comm, st)); CK(cudaStreamSynchronize(st)); };
  // first call (+ dump)
  align(); op(); CK(cudaStreamSynchronize(st));
  if (rank == 0 && !g.dump.empty()) {
    std::vector<uint16_t> ho(n); CK(cudaMemcpy(ho.data(), out, n * 2, cudaMemcpyDeviceToHost)); write_file(g.dump + ".out.bin", ho.data(), n * 2);
    if (norm) { CK(cudaMemcpy(ho.data(), res, n * 2, cudaMemcpyDeviceToHost)); write_file(g.dump + ".res_out.bin", ho.data(), n * 2); }
  }
  // graph of K calls
  cudaGraph_t graph; cudaGraphExec_t exec;
  align();
  CK(cudaStreamBeginCapture(st, cudaStreamCaptureModeRelaxed));
  for (int k = 0; k < g.graph; k++) { op_set(k); op(); }
  CK(cudaStreamEndCapture(st, &graph)); CK(cudaGraphInstantiate(&exec, graph, 0));
  for (int i = 0; i < g.warmup; i++) { align(); CK(cudaGraphLaunch(exec, st)); }
  cudaEvent_t e0, e1; CK(cudaEventCreate(&e0)); CK(cudaEventCreate(&e1));
  for (int i = 0; i < g.iters; i++) {
    align(); CK(cudaEventRecord(e0, st)); CK(cudaGraphLaunch(exec, st)); CK(cudaEventRecord(e1, st)); CK(cudaEventSynchronize(e1));
    float ms; CK(cudaEventElapsedTime(&ms, e0, e1)); g_times[rank][i] = ms;
  }
  if (g.e2e) {
    // one step end to end: pinned host -> device of one input set (and the residual), the K-call graph, 32 bytes back
    uint16_t *px = nullptr, *pr = nullptr, *po = nullptr;
    CK(cudaMallocHost(&px, n * 2)); memcpy(px, hx.data(), n * 2);
    if (norm) { CK(cudaMallocHost(&pr, n * 2)); memcpy(pr, hres.data(), n * 2); }
    CK(cudaMallocHost(&po, 32));
    if (rank == 0) { g_h2d = n * 2 * (norm ? 2 : 1); g_d2h = 32; }
    for (int i = 0; i < g.warmup + g.iters; i++) {
      align(); CK(cudaEventRecord(e0, st));
      CK(cudaMemcpyAsync(xset[0], px, n * 2, cudaMemcpyHostToDevice, st));
      if (norm) CK(cudaMemcpyAsync(res, pr, n * 2, cudaMemcpyHostToDevice, st));
      CK(cudaGraphLaunch(exec, st));
      CK(cudaMemcpyAsync(po, out, 32, cudaMemcpyDeviceToHost, st));
      CK(cudaEventRecord(e1, st)); CK(cudaEventSynchronize(e1));
      float ms; CK(cudaEventElapsedTime(&ms, e0, e1));
      if (i >= g.warmup) g_e2e[rank][i - g.warmup] = ms;
    }
  }
  CK(cudaStreamSynchronize(st)); bar->wait();
  if (norm) lnorm_fini(&ctx); else V->fini(&ctx);
}

int main(int argc, char** argv) {
  for (int i = 1; i + 1 < argc; i += 2) {
    std::string k = argv[i], v = argv[i + 1];
    if (k == "--tp") g.tp = atoi(v.c_str()); else if (k == "--rows") g.rows = atoi(v.c_str()); else if (k == "--variant") g.variant = v;
    else if (k == "--input") g.input = v; else if (k == "--epi") g.epi = atoi(v.c_str()); else if (k == "--algo") g.algo = atoi(v.c_str());
    else if (k == "--graph") g.graph = atoi(v.c_str()); else if (k == "--iters") g.iters = atoi(v.c_str()); else if (k == "--warmup") g.warmup = atoi(v.c_str());
    else if (k == "--nsets") g.nsets = std::max(1, atoi(v.c_str())); else if (k == "--mode") g.mode = atoi(v.c_str());
    else if (k == "--solo") g.solo = atoi(v.c_str()); else if (k == "--e2e") g.e2e = atoi(v.c_str());
    else if (k == "--in") g.in = v; else if (k == "--dump") g.dump = v; else { fprintf(stderr, "unknown flag %s\n", k.c_str()); return 2; }
  }
  int ndev = 0; CK(cudaGetDeviceCount(&ndev));
  if (g.mode < 0 || g.mode > 2) { fprintf(stderr, "--mode must be 0, 1 or 2\n"); return 2; }
  if (g.solo && g.mode != 2) { fprintf(stderr, "--solo 1 needs --mode 2: a rank launched alone would wait for peers that never run\n"); return 2; }
  if (g.tp < 2 || (!g.solo && g.tp > ndev) || ndev < 1 || (g.tp != 2 && g.tp != 4)) { printf("{\"impl\": \"reference\", \"unavailable\": \"reference push kernels support 2 or 4 ranks; asked for %d with %d GPUs visible\"}\n", g.tp, ndev); return 0; }
  if (g.variant != "L2" && g.variant != "L4" && g.variant != "lnorm") { fprintf(stderr, "variant must be L2, L4 or lnorm\n"); return 2; }
  if (g.input != "bf16" && g.input != "nvfp4") { fprintf(stderr, "--input must be bf16 or nvfp4\n"); return 2; }
  if (g.input == "nvfp4" && g.variant == "lnorm" && g.tp != 2) { printf("{\"impl\": \"reference\", \"unavailable\": \"the reference's fused norm kernel takes NVFP4 input at 2 ranks only\"}\n"); return 0; }
  size_t wb = g.variant == "lnorm" ? lnorm_window_bytes(g.rows, H, g.tp)
              : (g.variant == "L2" ? fp4ar_register_L2() : fp4ar_register_L4())->window_bytes(g.rows, H, g.tp);
  if (!wb) { printf("{\"impl\": \"reference\", \"unavailable\": \"variant %s has no window layout for %d ranks\"}\n", g.variant.c_str(), g.tp); return 0; }
  ncclUniqueId id; NK(ncclGetUniqueId(&id));
  const int nthreads = g.solo ? 1 : g.tp;
  HostBarrier bar(nthreads);
  std::vector<char*> windows(g.tp, nullptr);
  g_times.assign(nthreads, std::vector<float>(g.iters, 0.f));
  g_e2e.assign(nthreads, std::vector<float>(g.iters, 0.f));
  std::vector<std::thread> th;
  for (int r = 0; r < nthreads; r++) th.emplace_back(worker, r, id, &bar, &windows, wb);
  for (auto& t : th) t.join();
  auto per_call = [&](const std::vector<std::vector<float>>& t) {
    std::vector<float> mx(g.iters);
    for (int i = 0; i < g.iters; i++) { float m = 0; for (int r = 0; r < nthreads; r++) m = std::max(m, t[r][i]); mx[i] = m * 1000.f / g.graph; }
    std::sort(mx.begin(), mx.end());
    return mx;
  };
  const std::vector<float> mx = per_call(g_times);
  char e2e[256] = "";
  if (g.e2e) {
    const std::vector<float> ex = per_call(g_e2e);
    snprintf(e2e, sizeof(e2e), ", \"e2e_med_us\": %.3f, \"e2e_p10_us\": %.3f, \"e2e_p90_us\": %.3f, \"h2d_bytes_per_step\": %zu, \"d2h_bytes_per_step\": %zu",
             ex[g.iters / 2], ex[g.iters / 10], ex[(g.iters * 9) / 10], g_h2d, g_d2h);
  }
  printf("{\"impl\": \"reference\", \"variant\": \"%s\", \"input\": \"%s\", \"tp\": %d, \"rows\": %d, \"epi\": %d, \"graphK\": %d, \"iters\": %d, \"warmup\": %d, "
         "\"mode\": %d, \"solo\": %d, \"nsets\": %d, \"med_us\": %.3f, \"p10_us\": %.3f, \"p90_us\": %.3f, \"window_bytes\": %zu%s}\n",
         g.variant.c_str(), g.input.c_str(), g.tp, g.rows, g.epi, g.graph, g.iters, g.warmup, g.mode, g.solo, g.nsets,
         mx[g.iters / 2], mx[g.iters / 10], mx[(g.iters * 9) / 10], wb, e2e);
  fflush(stdout);
  _exit(0);   // the reference harness leaves the same way: NCCL / driver teardown can hang after graph capture
}
