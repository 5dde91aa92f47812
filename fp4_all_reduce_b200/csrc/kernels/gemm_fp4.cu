// Row-parallel GEMM with an NVFP4 epilogue that pushes straight into the AllReduce receive windows.
//
//   partial[M, N] = X[M, K] (BF16, K contiguous) x Wt[N, K]^T (BF16, K contiguous), FP32 accumulate
//   epilogue: every 16 consecutive outputs of a row are quantised with the static per-rank scale gs
//             (block scale e4m3(rn(rn(blockmax/gs')/6)), values e2m1, -0 canonicalised: the static-scale row
//             format of the AllReduce), and the row pieces are stored
//               - into every rank's receive window (one-shot), or into the row owner's window (two-shot),
//                 where the AllReduce kernel in "pushed input" mode finds them, and/or
//               - into a local [M, N/2 + N/16] NVFP4 tensor.
//
// sm_100a structure: persistent CTAs (one per SM), K in blocks of 64, three shapes:
//   pairs  (default for K >= 4096 or M >= 8192): the two CTAs of a cluster share one 256 x 256 tile with tcgen05
//          cta_group::2: each loads its own 128 rows of A and half of the B block into a 6-stage ring, the even CTA
//          issues the MMAs for both, each CTA's TMEM holds the accumulator of its own 128 rows;
//   single: one CTA per 128 x 256 tile (4-stage ring) or 128 x 192 tile (5-stage ring, where that fills the last wave
//          of CTAs better and the K split below does not apply).
// Where the tile count is not a multiple of the unit count (CTAs or pairs), the first (units + remainder) tiles are cut
// along K into equal ranges per unit (stream-K, see SegIter) so that no SM idles through a last wave.
//   warp 0  : TMA producer   - cp.async.bulk.tensor (every CTA loads for itself) of the A and B blocks into the ring,
//                              128-byte swizzle, completion on mbarriers (of a pair: both CTAs' bytes are counted
//                              under the leader's barrier)
//   warp 1  : MMA issuer     - one thread issues tcgen05.mma (kind::f16, M 128 per CTA, N 256, K 16) from
//                              shared-memory descriptors into TMEM; tcgen05.commit releases ring stages and
//                              publishes finished accumulators (of a pair: on both CTAs' barriers); owns
//                              tcgen05.alloc / dealloc (512 columns = two accumulators, so the epilogue of tile i
//                              overlaps the main loop of tile i+1)
//   warps 2-5: epilogue      - tcgen05.ld (32 lanes x 32 columns per instruction), quantise, stage the row
//                              pieces in shared memory, bulk-store them to the (peer) windows
// Every wait is bounded; a wait that gives up raises a CTA-wide abort flag, the roles drain, TMEM is freed and
// the status word reports it.
//
// The reference project has no such producer: its NVFP4-input kernels assume one and the harness emulates it
// with a copy (README.md:76, docs/INTEGRATION.md:67-74, harness/fp4ar_bench.cu:205-215).
#include <cuda.h>
#include <cuda_runtime.h>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include "../include/fp4ar.h"
#include "../include/fp4ar_codec.cuh"
#include "../include/fp4ar_async.cuh"
#include "../include/fp4ar_gemm.h"
#include "host_util.h"

namespace fp4ar {

constexpr int kBM = 128, kBK = 64;
constexpr int kABytes = kBM * kBK * 2;            // 16 KB
constexpr int kGemmThreads = 192;
constexpr uint32_t kTmemCols = 512;
constexpr int kMaxStages = 6;

// Tile width BN: 256 with a 4-stage ring, or 192 with a 5-stage ring.  With 148 persistent CTAs the tile count decides
// how full the last wave is: M = 1024, N = 6144 gives 192 tiles of 128 x 256 (1.3 waves, 65 % busy) but 256 tiles of
// 128 x 192 (1.7 waves, 86 % busy).  (A 128-wide tile with a 6-stage ring was measured 15-35 % slower at every M from
// 1024 to 4096 and is not built.)
// G = 2: two CTAs of a cluster (an SM pair) work on one 256 x 256 tile with tcgen05 cta_group::2: each CTA loads its own
// 128 rows of A and HALF of the B block (128 of the 256 columns), the tensor cores of both SMs read both halves, and
// each CTA's TMEM holds the accumulator of its own 128 rows.  A K block then costs a CTA 32 KB of shared-memory fill
// instead of 48 KB, and the ring is six stages deep.
template <int BN, int G = 1>
struct GemmShape {
  static_assert(BN == 256 || BN == 192, "tile width");
  static_assert(G == 1 || (G == 2 && BN == 256), "CTA pairs use the 256-wide tile");
  static constexpr int kStages = G == 2 ? 6 : (BN == 256 ? 4 : 5);
  static constexpr int kBBytes = BN / G * kBK * 2;              // 32 KB / 24 KB, 16 KB per CTA of a pair
  static constexpr int kStageBytes = kABytes + kBBytes;         // 48 KB / 40 KB / 32 KB
  static constexpr int kTxBytes = kStageBytes * G;              // what lands per stage under the (leader's) full barrier
  static constexpr int kValueB = BN / 2, kScaleB = BN / 16;     // 128 + 16 B / 96 + 12 B of one row of one tile
  static constexpr int kPieceBytes = (kValueB + kScaleB + 15) & ~15;   // 144 / 112: keeps every piece 16-byte aligned
  static constexpr int kEpiBytes = kBM * kPieceBytes;
  static constexpr int kSmem = kStages * kStageBytes + kEpiBytes + 256 + 1024;   // + barriers + alignment slack
  // Instruction descriptor: D = F32, A = B = BF16, both K-major, N = BN, M = 128 per CTA of the group.
  static constexpr uint32_t kIdesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)((kBM * G) >> 4) << 24);
};

struct GemmParams {
  int M, N, K;
  float inv_gs;
  // push destination (nranks == 0: none)
  char* win[kMaxRanksOps];
  const uint32_t* call_counter;
  unsigned long long buf_bytes;
  int cap, capo, nranks, rank, two_shot;
  // local outputs (optional)
  char* local_q;       // [M][N/2 + N/16]
  float* dbg_acc;      // [M][N]
  StatusWords* status;
  unsigned long long timeout_ns;
  // split of the K loop across CTAs (see SegIter): partial accumulators and their flags, one slot per CTA
  int stream_k;
  float* sk_partial;     // [grid][BN / 32][8][128] float4
  uint32_t* sk_flags;    // [grid][4]: 1 = the slot's quarter (32 rows) is written and not yet consumed
};

// ---- tcgen05 / TMA wrappers ----
__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
               ::"r"(smem_addr(smem_dst)), "l"(map), "r"(x), "r"(y), "r"(smem_addr(bar))
               : "memory");
}
__device__ __forceinline__ void tmem_alloc(uint32_t* holder, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_addr(holder)), "r"(cols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() { asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_dealloc(uint32_t addr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(addr), "r"(cols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void umma_bf16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  asm volatile("{ .reg .pred p;\n"
               "  setp.ne.b32 p, %4, 0;\n"
               "  tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p; }"
               ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
               : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_addr(bar)) : "memory");
}
// ---- CTA pair (cluster of two) ----
__device__ __forceinline__ uint32_t cluster_cta_rank() { uint32_t r; asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r)); return r; }
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// shared::cluster address of the same shared-memory location in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t cluster_addr(const void* local, uint32_t rank) {
  uint32_t a;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(a) : "r"(smem_addr(local)), "r"(rank));
  return a;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_bar) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_bar) : "memory");
}
// TMA load of one CTA of a pair: the bytes are counted under the barrier at `cluster_bar` (the leader's); every CTA loads for itself
__device__ __forceinline__ void tma_load_2d_pair(void* smem_dst, const CUtensorMap* map, int x, int y, uint32_t cluster_bar) {
  asm volatile("cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
               ::"r"(smem_addr(smem_dst)), "l"(map), "r"(x), "r"(y), "r"(cluster_bar)
               : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t* holder, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_addr(holder)), "r"(cols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() { asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t addr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(addr), "r"(cols) : "memory");
}
__device__ __forceinline__ void umma_bf16_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  asm volatile("{ .reg .pred p;\n"
               "  setp.ne.b32 p, %4, 0;\n"
               "  tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p; }"
               ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
               : "memory");
}
// arrives on the barrier at the same shared-memory offset in both CTAs of the pair once the MMAs issued so far are done
__device__ __forceinline__ void umma_commit_pair(uint64_t* bar) {
  asm volatile("{ .reg .b16 m;\n"
               "  mov.b16 m, 3;\n"
               "  tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], m; }"
               ::"r"(smem_addr(bar)) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.release.cta.shared::cta.b64 _, [%0];" ::"r"(smem_addr(bar)) : "memory");
}
// Starts the load of 32 accumulator columns of this thread's TMEM lane; the registers are valid after tmem_ld_wait().
__device__ __forceinline__ void tmem_ld32_issue(uint32_t taddr, float* v) {
  uint32_t* r = reinterpret_cast<uint32_t*>(v);
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 "
               "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
               "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                 "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
                 "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
                 "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
               : "r"(taddr));
}
// All tcgen05.ld of this thread issued so far have delivered their registers.
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor of a K-major tile whose rows are 128 bytes (64 BF16) with the 128-byte
// swizzle: 8-row groups 1024 bytes apart, descriptor version 1 (sm_100), layout type 2 (SWIZZLE_128B).
__device__ __forceinline__ uint64_t umma_desc_k128(const void* smem_tile) {
  uint64_t d = (uint64_t)((smem_addr(smem_tile) >> 4) & 0x3FFFu);
  d |= (uint64_t)1 << 16;            // leading byte offset (unused with a swizzle), in 16-byte units
  d |= (uint64_t)(1024 >> 4) << 32;  // stride byte offset between 8-row groups
  d |= (uint64_t)1 << 46;            // version
  d |= (uint64_t)2 << 61;            // SWIZZLE_128B
  return d;
}

// Tile order: the N tiles are walked in panels of kPanel; inside a panel consecutive tile indices step through
// N fastest and then M.  The ~148 tiles in flight at a time then cover about 18 row blocks x 8 column tiles, which
// needs (18 + 2*8) * 128 * K * 2 bytes of operands from L2 instead of (6 + 2*24) for a plain row-major walk.
constexpr int kPanel = 8;
template <int BN, int G = 1>
__device__ __forceinline__ void tile_coords(int t, int m_tiles, int n_tiles, int& m0, int& n0) {
  const int per_panel = m_tiles * kPanel;
  const int panel = t / per_panel, within = t - panel * per_panel;
  const int width = min(kPanel, n_tiles - panel * kPanel);
  const int m = within / width, n = panel * kPanel + within % width;
  m0 = m * kBM * G; n0 = n * BN;
}

struct GemmWait {
  volatile uint32_t* abort_flag;
  StatusWords* status;
  unsigned long long limit_ns;
};
// Bounded mbarrier wait; false when it gave up or the CTA is aborting.
__device__ __forceinline__ bool gemm_wait(uint64_t* bar, uint32_t parity, const GemmWait& w, uint32_t what) {
  if (mbar_test(bar, parity)) return true;
  const unsigned long long t0 = global_timer_ns();
  uint32_t n = 0;
  while (!mbar_test(bar, parity)) {
    if ((++n & 255u) == 0u) {
      if (*w.abort_flag) return false;
      if (global_timer_ns() - t0 > w.limit_ns) {
        *w.abort_flag = 1u;
        if (atomicCAS(&w.status->code, 0u, (uint32_t)kStatusLoadTimeout) == 0u) { w.status->detail = 16u + what; w.status->cta = blockIdx.x; }
        atomicAdd(&w.status->count, 1u);
        return false;
      }
    }
  }
  return true;
}

// Bounded wait until *flag == want (acquire); false when it gave up or the CTA is aborting.
__device__ __forceinline__ uint32_t ld_acquire_gpu(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.gpu.global.b32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_gpu(uint32_t* p, uint32_t v) {
  asm volatile("st.release.gpu.global.b32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ bool gemm_flag_wait(const uint32_t* flag, uint32_t want, const GemmWait& w, uint32_t what) {
  if (ld_acquire_gpu(flag) == want) return true;
  const unsigned long long t0 = global_timer_ns();
  uint32_t n = 0;
  while (ld_acquire_gpu(flag) != want) {
    if ((++n & 63u) == 0u) {
      if (*w.abort_flag) return false;
      if (global_timer_ns() - t0 > w.limit_ns) {
        *w.abort_flag = 1u;
        if (atomicCAS(&w.status->code, 0u, (uint32_t)kStatusLoadTimeout) == 0u) { w.status->detail = 16u + what; w.status->cta = blockIdx.x; }
        atomicAdd(&w.status->count, 1u);
        return false;
      }
    }
  }
  return true;
}

// The work of one CTA as a list of segments (tile, K blocks [lo, lo + count), rotation), the same list in all three roles.
//   plain:    whole tiles blockIdx.x, blockIdx.x + grid, ...
//   stream-K: with tiles = w * grid + r (0 < r < grid) the first grid + r tiles are cut, as tiles x kblocks units,
//             into `grid` equal contiguous ranges, so every CTA runs the same number of K blocks there (between one and
//             two tiles' worth) instead of r CTAs running one more tile than the others; the other (w - 1) * grid
//             tiles follow as whole tiles.  A range is at least one tile long, so a tile is shared by at most two
//             CTAs: the one whose range BEGINS inside the tile (kProduce) runs its share first, on the tile's FIRST K
//             blocks, and leaves its FP32 accumulator in its slot of the partial buffer; the one whose range ENDS
//             inside the tile (kFix) runs the remaining K blocks last, adds that partial and does the tile's epilogue.
//             The partial was written about one tile duration or more before it is read.
//   K order:  every segment walks its K blocks upwards.  The producing share is the tile's FIRST K blocks and the fixing
//             share its LAST ones, so a CTA that starts with a share of c blocks is at block t while it produces, at
//             t - c in the whole tile that follows and at most (range - kblocks) behind t in its fixing share: at
//             any moment all CTAs read 64-column slices of X and Wt that lie within that window of each other and no
//             slice is needed again after the window has passed, so the operands cross HBM once.  (Shares that start
//             at unrelated K offsets: 123 us at M = 1024, K = 8192; a cyclic walk locked to a common clock: 94 us,
//             267 MB of DRAM reads for 116 MB of operands because the wrapped part is re-read.)
enum : int { kWhole = 0, kProduce = 1, kFix = 2 };
struct Seg { int tile, lo, count, kind; };      // K blocks lo .. lo + count - 1
struct SegIter {
  int tiles, kblocks, stride, t;
  long long u, u_end;
  // unit = this CTA (or CTA pair) among `units` of them
  __host__ __device__ SegIter(int stream_k, int tiles_, int kblocks_, int unit, int units) : tiles(tiles_), kblocks(kblocks_), stride(units) {
    const int g = units;
    const int cut_tiles = stream_k ? g + tiles_ % g : 0;
    const long long total = (long long)cut_tiles * kblocks_;
    u = total * unit / g;
    u_end = total * (unit + 1) / g;
    t = cut_tiles + unit;
  }
  __host__ __device__ bool next(Seg& s) {
    if (u < u_end) {
      s.tile = (int)(u / kblocks);
      const int off = (int)(u - (long long)s.tile * kblocks);
      const long long left = u_end - u;
      const int room = kblocks - off;
      s.count = (int)(left < room ? left : room);
      if (off > 0) { s.kind = kProduce; s.lo = 0; }
      else if (s.count < kblocks) { s.kind = kFix; s.lo = kblocks - s.count; }
      else { s.kind = kWhole; s.lo = 0; }
      u += s.count;
    } else {
      if (t >= tiles) return false;
      s.tile = t; s.lo = 0; s.count = kblocks; s.kind = kWhole;
      t += stride;
    }
    return true;
  }
};

template <int BN, int G>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_nvfp4_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                  const __grid_constant__ GemmParams p) {
  using S = GemmShape<BN, G>;
  constexpr int kStages = S::kStages, kStageBytes = S::kStageBytes, kEpiBytes = S::kEpiBytes, kPieceBytes = S::kPieceBytes;
  constexpr uint32_t kIdesc = S::kIdesc;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* ring = smem;
  uint8_t* epi = smem + kStages * kStageBytes;
  uint64_t* full = reinterpret_cast<uint64_t*>(epi + kEpiBytes);   // [kMaxStages]
  uint64_t* empty = full + kMaxStages;                              // [kMaxStages]
  uint64_t* acc_full = empty + kMaxStages;                          // [2]
  uint64_t* acc_empty = acc_full + 2;                               // [2]
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile uint32_t* abort_flag = tmem_holder + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_tiles = p.N / BN, m_tiles = (p.M + kBM * G - 1) / (kBM * G);
  const int tiles = n_tiles * m_tiles, kblocks = p.K / kBK;
  // a pair works as one unit: the even CTA (cluster rank 0) leads, i.e. owns the barriers the MMAs wait on and issues them
  const uint32_t crank = G == 2 ? cluster_cta_rank() : 0u;
  const bool leads = crank == 0u;
  const int unit = blockIdx.x / G, units = gridDim.x / G;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; s++) { mbar_init(full + s, 1); mbar_init(empty + s, 1); }
    for (int a = 0; a < 2; a++) { mbar_init(acc_full + a, 1); mbar_init(acc_empty + a, 128 * G); }
    *abort_flag = 0u;
    mbar_init_fence();
  }
  if (warp == 1) {
    if constexpr (G == 2) { tmem_alloc_pair(tmem_holder, kTmemCols); tmem_relinquish_pair(); }
    else { tmem_alloc(tmem_holder, kTmemCols); tmem_relinquish(); }
  }
  tc_fence_before();
  __syncthreads();
  if constexpr (G == 2) cluster_sync_all();     // the partner's barriers exist before anything arrives on them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;
  GemmWait gw{abort_flag, p.status, p.timeout_ns};

  pdl_wait_prior_grids();   // the windows and the call counter belong to the previous kernel until here
  pdl_release_dependents();

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      uint32_t it = 0;
      SegIter seg(p.stream_k, tiles, kblocks, unit, units);
      Seg sg;
      while (seg.next(sg)) {
        int m0, n0;
        tile_coords<BN, G>(sg.tile, m_tiles, n_tiles, m0, n0);
        for (int j = 0; j < sg.count; j++, it++) {
          const int kb = sg.lo + j;
          const int s = it % kStages;
          if (!gemm_wait(empty + s, ((it / kStages) & 1u) ^ 1u, gw, 1)) {
            // giving up: let the loads already issued land before the CTA (and its shared memory) goes away
            if (leads) {
              for (uint32_t back = 1; back <= (uint32_t)kStages && back <= it; back++) {
                const uint32_t j = it - back;
                uint32_t spins = 0;
                while (!mbar_test(full + (j % kStages), (j / kStages) & 1u) && ++spins < (1u << 20)) {}
              }
            } else {
              for (int w = 0; w < 2000; w++) __nanosleep(1000);   // its loads complete under the leader's barriers: 2 ms
            }
            goto done;
          }
          if constexpr (G == 2) {
            // both CTAs' bytes are counted under the leader's barrier; only the leader announces them
            const uint32_t lead_full = cluster_addr(full + s, 0u);
            if (leads) mbar_arrive_expect(full + s, S::kTxBytes);
            tma_load_2d_pair(ring + s * kStageBytes, &map_a, kb * kBK, m0 + (int)crank * kBM, lead_full);
            tma_load_2d_pair(ring + s * kStageBytes + kABytes, &map_b, kb * kBK, n0 + (int)crank * (BN / 2), lead_full);
          } else {
            mbar_arrive_expect(full + s, kStageBytes);
            tma_load_2d(ring + s * kStageBytes, &map_a, kb * kBK, m0, full + s);
            tma_load_2d(ring + s * kStageBytes + kABytes, &map_b, kb * kBK, n0, full + s);
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer (of a pair: the leader's)
    if (lane == 0 && leads) {
      uint32_t it = 0, tile_i = 0;
      SegIter seg(p.stream_k, tiles, kblocks, unit, units);
      Seg sg;
      for (; seg.next(sg); tile_i++) {
        const uint32_t a = tile_i & 1u;
        if (!gemm_wait(acc_empty + a, ((tile_i >> 1) & 1u) ^ 1u, gw, 2)) goto done;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + a * BN;
        for (int j = 0; j < sg.count; j++, it++) {
          const int s = it % kStages;
          if (!gemm_wait(full + s, (it / kStages) & 1u, gw, 3)) goto done;
          tc_fence_after();
          const uint64_t da = umma_desc_k128(ring + s * kStageBytes);
          const uint64_t db = umma_desc_k128(ring + s * kStageBytes + kABytes);
#pragma unroll
          for (int k = 0; k < kBK / 16; k++) {
            if constexpr (G == 2) umma_bf16_pair(d_tmem, da + (uint64_t)(2 * k), db + (uint64_t)(2 * k), kIdesc, (j | k) != 0 ? 1u : 0u);
            else umma_bf16(d_tmem, da + (uint64_t)(2 * k), db + (uint64_t)(2 * k), kIdesc, (j | k) != 0 ? 1u : 0u);
          }
          // the stage is free once these MMAs have read it (of a pair: in both CTAs)
          if constexpr (G == 2) umma_commit_pair(empty + s); else umma_commit(empty + s);
        }
        // the accumulator is complete once everything above has run
        if constexpr (G == 2) umma_commit_pair(acc_full + a); else umma_commit(acc_full + a);
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue (warps 2..5 = 128 threads = 128 rows)
    const int q = warp & 3;                       // TMEM lane quarter this warp may read
    const int r_in_tile = q * 32 + lane;
    uint8_t* my_piece = epi + r_in_tile * kPieceBytes;
    const size_t buf_off = p.nranks ? (size_t)(*p.call_counter & 1u) * p.buf_bytes : 0;
    const int qrow_bytes = p.N / 2 + p.N / 16;
    uint32_t tile_i = 0;
    SegIter seg(p.stream_k, tiles, kblocks, unit, units);
    Seg sg;
    // this thread's float4 i of chunk c inside a partial slot: a warp's 32 rows are 512 contiguous bytes
    auto slot_ptr = [&](int cta, int c, int i) {
      return reinterpret_cast<float4*>(p.sk_partial) + ((size_t)cta * (BN / 32) + c) * 8 * kBM + (size_t)i * kBM + r_in_tile;
    };
    // 128 arrivals per CTA hand the accumulator back to the MMA warp (of a pair: to the leader's)
    auto hand_back = [&](uint32_t a) {
      if constexpr (G == 2) mbar_arrive_cluster(cluster_addr(acc_empty + a, 0u)); else mbar_arrive(acc_empty + a);
    };
    for (; seg.next(sg); tile_i++) {
      int m0, n0;
      tile_coords<BN, G>(sg.tile, m_tiles, n_tiles, m0, n0);
      m0 += (int)crank * kBM;                              // of a pair: this CTA's half of the 256 rows
      const uint32_t a = tile_i & 1u;
      const int row = m0 + r_in_tile;
      const bool produces = sg.kind == kProduce;           // a share of the tile's K blocks: leave a partial
      const bool fixes = sg.kind == kFix;                  // the rest of them: add the next CTA's partial
      const uint32_t tbase = tmem_base + ((uint32_t)(q * 32) << 16) + a * BN;
      if (produces) {
        // the slot is free once the consumer of an earlier launch has reset the flag
        uint32_t* flag = p.sk_flags + blockIdx.x * 4 + q;
        bool ok = lane == 0 ? gemm_flag_wait(flag, 0u, gw, 5) : true;
        ok = __all_sync(0xffffffffu, ok) && __all_sync(0xffffffffu, gemm_wait(acc_full + a, (tile_i >> 1) & 1u, gw, 4));
        if (!ok) break;
        tc_fence_after();
        float v[2][32];
        tmem_ld32_issue(tbase, v[0]);
#pragma unroll
        for (int c = 0; c < BN / 32; c++) {
          tmem_ld_wait();
          if (c + 1 < BN / 32) tmem_ld32_issue(tbase + (c + 1) * 32, v[(c + 1) & 1]);
          const float* vc = v[c & 1];
#pragma unroll
          for (int i = 0; i < 8; i++) *slot_ptr(blockIdx.x, c, i) = make_float4(vc[4 * i], vc[4 * i + 1], vc[4 * i + 2], vc[4 * i + 3]);
        }
        tc_fence_before();
        hand_back(a);
        __syncwarp();
        if (lane == 0) { __threadfence(); st_release_gpu(flag, 1u); }
        continue;
      }
      float pv[2][32];
      uint32_t* fix_flag = p.sk_flags + (blockIdx.x + G) * 4 + q;
      auto load_partial = [&](int c, float* dst) {
#pragma unroll
        for (int i = 0; i < 8; i++) {
          const float4 f = __ldcg(slot_ptr(blockIdx.x + G, c, i));
          dst[4 * i] = f.x; dst[4 * i + 1] = f.y; dst[4 * i + 2] = f.z; dst[4 * i + 3] = f.w;
        }
      };
      if (fixes) {
        // written about one kernel duration ago; fetched while the last K blocks of this tile are still running
        bool ok = lane == 0 ? gemm_flag_wait(fix_flag, 1u, gw, 6) : true;
        if (!__all_sync(0xffffffffu, ok)) break;
        load_partial(0, pv[0]);
      }
      // warp-uniform verdict: the tcgen05.ld below is a warp-wide instruction
      if (!__all_sync(0xffffffffu, gemm_wait(acc_full + a, (tile_i >> 1) & 1u, gw, 4))) break;
      tc_fence_after();
      bulk_wait_source_free<0>();   // this thread's previous pieces have left its staging row
      // 32 columns at a time, double-buffered: the load of chunk c + 1 is in flight while chunk c is quantised
      float v[2][32];
      tmem_ld32_issue(tbase, v[0]);
#pragma unroll
      for (int c = 0; c < BN / 32; c++) {
        tmem_ld_wait();
        if (c + 1 < BN / 32) tmem_ld32_issue(tbase + (c + 1) * 32, v[(c + 1) & 1]);
        float* vc = v[c & 1];
        if (fixes) {
          if (c + 1 < BN / 32) load_partial(c + 1, pv[(c + 1) & 1]);
          const float* pc = pv[c & 1];
#pragma unroll
          for (int i = 0; i < 32; i++) vc[i] = __fadd_rn(vc[i], pc[i]);
        }
        if (p.dbg_acc && row < p.M) {
          float4* dst = reinterpret_cast<float4*>(p.dbg_acc + (size_t)row * p.N + n0 + c * 32);
#pragma unroll
          for (int i = 0; i < 8; i++) dst[i] = make_float4(vc[4 * i], vc[4 * i + 1], vc[4 * i + 2], vc[4 * i + 3]);
        }
        uint4 qv;
        const uint32_t sf2 = encode_pair_f32<true>(vc, [&](float b0, float b1, float& m0, float& m1) {
          return pair_block_scales(b0, b1, p.inv_gs, m0, m1);
        }, qv);
        *reinterpret_cast<uint4*>(my_piece + 16 * c) = qv;
        *reinterpret_cast<uint16_t*>(my_piece + S::kValueB + 2 * c) = (uint16_t)sf2;
      }
      if (fixes) {
        __syncwarp();
        if (lane == 0) st_release_gpu(fix_flag, 0u);        // every lane has its partial in registers: the slot is free
      }
      tc_fence_before();
      hand_back(a);                 // 128 arrivals hand the accumulator back to the MMA warp
      fence_smem_to_async();
      if (row < p.M) {
        const size_t voff = (size_t)(n0 / 2), soff = (size_t)(p.N / 2 + n0 / 16);
        // one row piece to one destination row: the values by a bulk store; the scales by a bulk store when they are
        // a 16-byte granule (BN = 256), else (12 bytes at a 4-byte aligned offset) by three word stores from registers
        auto put = [&](char* dst) {
          bulk_store(dst + voff, my_piece, S::kValueB);
          if constexpr (S::kScaleB == 16) {
            bulk_store(dst + soff, my_piece + S::kValueB, 16);
          } else {
            const uint32_t* sw = reinterpret_cast<const uint32_t*>(my_piece + S::kValueB);
            uint32_t* dw = reinterpret_cast<uint32_t*>(dst + soff);
#pragma unroll
            for (int i = 0; i < S::kScaleB / 4; i++) dw[i] = sw[i];
          }
        };
        if (p.local_q) put(p.local_q + (size_t)row * qrow_bytes);
        if (p.nranks) {
          if (p.two_shot) {
            put(p.win[row % p.nranks] + buf_off + ((size_t)p.rank * p.capo + row / p.nranks) * kRecStride);
          } else {
            for (int d = 0; d < p.nranks; d++) put(p.win[d] + buf_off + ((size_t)p.rank * p.cap + row) * kRecStride);
          }
        }
      }
      bulk_commit();
      __syncwarp();
    }
    bulk_wait_done<0>();
  }
done:
  tc_fence_before();
  __syncthreads();
  if constexpr (G == 2) cluster_sync_all();   // neither CTA frees TMEM or leaves while the other's MMAs, commits or arrivals may still touch it
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    if constexpr (G == 2) tmem_dealloc_pair(tmem_base, kTmemCols); else tmem_dealloc(tmem_base, kTmemCols);
  }
}

// ---- host side ----
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}
static bool make_map(CUtensorMap* m, const void* base, int rows, int k, int box_rows) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return false;
  cuuint64_t dims[2] = {(cuuint64_t)k, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)k * 2};
  cuuint32_t box[2] = {(cuuint32_t)kBK, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  return fn(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

static StatusWords* gemm_status_word() {
  static StatusWords* p[64] = {nullptr};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  if (!p[dev]) {
    if (cudaMalloc(&p[dev], sizeof(StatusWords)) != cudaSuccess) return nullptr;
    cudaMemset(p[dev], 0, sizeof(StatusWords));
  }
  return p[dev];
}

// Partial accumulators of the stream-K split: one slot of 128 x 256 floats and four flags per SM, allocated at the
// first call on a device and kept (19 MB on a B200).  Launches that share a device take turns on a slot through its
// flags: a producer waits until the consumer of the previous launch has reset them.
struct StreamKSpace { float* partial; uint32_t* flags; int slots; };
static StreamKSpace g_stream_k_space[64] = {};
static std::mutex g_stream_k_mu;
static bool stream_k_space(int slots, StreamKSpace* out) {
  StreamKSpace* sp = g_stream_k_space;
  std::mutex& mu = g_stream_k_mu;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return false;
  std::lock_guard<std::mutex> g(mu);
  if (!sp[dev].partial) {
    float* part = nullptr;
    uint32_t* fl = nullptr;
    const size_t pbytes = (size_t)slots * kBM * 256 * sizeof(float), fbytes = (size_t)slots * 4 * sizeof(uint32_t);
    if (cudaMalloc(&part, pbytes) != cudaSuccess) { cudaGetLastError(); return false; }
    if (cudaMalloc(&fl, fbytes) != cudaSuccess) { cudaGetLastError(); cudaFree(part); return false; }
    if (cudaMemset(fl, 0, fbytes) != cudaSuccess) { cudaGetLastError(); cudaFree(part); cudaFree(fl); return false; }
    sp[dev] = StreamKSpace{part, fl, slots};
  }
  if (sp[dev].slots < slots) return false;
  *out = sp[dev];
  return true;
}

}  // namespace fp4ar

using namespace fp4ar;

// Which shape a call takes.  `units` = CTAs (or CTA pairs) that work, `tiles` = output tiles of that shape.
struct GemmPlan { int pair, bn, stream_k, units, tiles; };
static GemmPlan plan_gemm(int M, int N, int K, int sms, bool env) {
  // Tile width of single CTAs: the one whose tiles keep the persistent CTAs busier over all waves.  A 192-wide tile was
  // measured at about 0.87 of the per-cycle work of a 256-wide one (M = 4096: 321 vs 315 us at K = 8192 although its
  // last wave is full), so it is only taken where it wins clearly (M = 1024: 111 vs 123 us); N must be a multiple of
  // 192 too.  FP4AR_GEMM_TILE_N = 192 / 256 forces it (and single CTAs).
  int bn = 256;
  bool stream_k = false, pair = false;
  const char* force = env ? std::getenv("FP4AR_GEMM_TILE_N") : nullptr;
  const char* fsk = env ? std::getenv("FP4AR_GEMM_STREAM_K") : nullptr;
  const char* fp = env ? std::getenv("FP4AR_GEMM_PAIR") : nullptr;
  auto busy = [&](int w) {
    const long tiles = (long)(N / w) * ((M + kBM - 1) / kBM);
    return (double)tiles / (double)(((tiles + sms - 1) / sms) * sms);
  };
  if (N % 192 == 0 && 0.80 * busy(192) > busy(256)) bn = 192;
  if (force && std::atoi(force) == 256) bn = 256;
  if (force && std::atoi(force) == 192 && N % 192 == 0) bn = 192;
  // Stream-K (256-wide tiles, the K loop cut into equal ranges per CTA) where whole tiles would leave the last wave
  // of CTAs partly idle and the K loop is long enough to pay for the partial sums (K = 2048: 36.9 us against 33.0 us
  // with whole 192-wide tiles at M = 1024, level at M = 2048, 77.8 against 79.9 at M = 4096; K = 8192: 86 / 143 /
  // 264 us against 96 / 154 / 296 at M = 1024 / 2048 / 4096); FP4AR_GEMM_STREAM_K = 0 / 1 overrides.
  const long tiles256 = (long)(N / 256) * ((M + kBM - 1) / kBM);
  stream_k = tiles256 > sms && tiles256 % sms != 0 && busy(256) < 0.95 && (K >= 4096 || tiles256 >= 4 * sms) &&
             !(force && std::atoi(force) == 192);
  if (fsk) stream_k = std::atoi(fsk) != 0 && tiles256 > sms && tiles256 % sms != 0;
  if (stream_k) bn = 256;
  // CTA pairs (tcgen05 cta_group::2) where the K loop is long or there are many tiles: measured against single CTAs
  // at M = 1024 / 2048 / 4096 / 16384: K = 8192: 80 / 131 / 252 / 1054 us against 88 / 143 / 268 / 1078; K = 4096:
  // 52 / 76 / 135 / 506 against 53 / 78 / 137 / 524; K = 2048: 35 / 49 / 80 / 260 against 33 / 47 / 78 / 266.
  // FP4AR_GEMM_PAIR = 0 / 1 overrides.
  const bool want_pair = fp ? std::atoi(fp) != 0 : ((K >= 4096 || M >= 8192) && !force);
  long tiles = (long)(N / bn) * ((M + kBM - 1) / kBM);
  int units = sms;
  if (want_pair && sms >= 2) {
    pair = true; bn = 256;
    units = sms / 2;
    tiles = (long)(N / 256) * ((M + 2 * kBM - 1) / (2 * kBM));
    const double busy2 = (double)tiles / (double)(((tiles + units - 1) / units) * units);
    stream_k = tiles > units && tiles % units != 0 && busy2 < 0.95 && (K >= 4096 || tiles >= 4 * units);
    if (fsk) stream_k = std::atoi(fsk) != 0 && tiles > units && tiles % units != 0;
  }
  if (tiles < units) units = (int)tiles;
  return GemmPlan{pair ? 1 : 0, bn, stream_k ? 1 : 0, units, (int)tiles};
}

template <int BN, int G>
static int launch_gemm(const CUtensorMap& ma, const CUtensorMap& mb, GemmParams p, cudaStream_t stream) {
  using S = GemmShape<BN, G>;
  if (cudaFuncSetAttribute(gemm_nvfp4_kernel<BN, G>, cudaFuncAttributeMaxDynamicSharedMemorySize, S::kSmem) != cudaSuccess) return cuda_fail();
  const int tiles = (p.N / BN) * ((p.M + kBM * G - 1) / (kBM * G));
  const int sms = device_sm_count();
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.blockDim = dim3(kGemmThreads);
  cfg.dynamicSmemBytes = S::kSmem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  int units = sms / G;
  cfg.attrs = attr;
  if (G == 2) {
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    cfg.numAttrs = 1;
    cfg.gridDim = dim3(sms & ~1);
    int clusters = 0;      // pairs that can be resident together: the grid is persistent, every pair must be
    if (cudaOccupancyMaxActiveClusters(&clusters, gemm_nvfp4_kernel<BN, G>, &cfg) != cudaSuccess || clusters < 1) return cuda_fail();
    if (clusters < units) units = clusters;
  }
  // Programmatic dependent launch: a CTA may start (barrier set-up, TMEM allocation) on an SM that the previous
  // kernel's CTA has left while other CTAs of that kernel still run; it touches global memory only after
  // griddepcontrol.wait.  FP4AR_GEMM_PDL = 0 turns it off.
  {
    const char* e = std::getenv("FP4AR_GEMM_PDL");
    if (!e || std::atoi(e) != 0) {
      attr[cfg.numAttrs].id = cudaLaunchAttributeProgrammaticStreamSerialization;
      attr[cfg.numAttrs].val.programmaticStreamSerializationAllowed = 1;
      cfg.numAttrs++;
    }
  }
  if (tiles < units) units = tiles;
  if (p.stream_k && (tiles <= units || tiles % units == 0)) p.stream_k = 0;      // fewer units fit than planned: whole tiles (see SegIter)
  cfg.gridDim = dim3(units * G);
  if (cudaLaunchKernelEx(&cfg, gemm_nvfp4_kernel<BN, G>, ma, mb, p) != cudaSuccess) return cuda_fail();
  return cuda_check_launch();
}

extern "C" int fp4ar_gemm_nvfp4(const fp4ar_push_view* push, int two_shot, const void* x, const void* wt, int M, int N,
                                int K, float gs, void* local_q, float* dbg_acc, fp4ar_stream stream) {
  if (!x || !wt || M < 1 || N < 256 || K < kBK || (N % 256) || (K % kBK) || !(gs > 0.0f)) return FP4AR_ERR_ARGUMENT;
  if (((uintptr_t)x | (uintptr_t)wt | (uintptr_t)local_q | (uintptr_t)dbg_acc) & 15) return FP4AR_ERR_ARGUMENT;
  if (!push && !local_q && !dbg_acc) return FP4AR_ERR_ARGUMENT;
  const GemmPlan pl = plan_gemm(M, N, K, device_sm_count(), /*env=*/true);
  const int bn = pl.bn;
  const bool stream_k = pl.stream_k != 0, pair = pl.pair != 0;
  GemmParams p;
  memset(&p, 0, sizeof(p));
  p.M = M; p.N = N; p.K = K; p.inv_gs = 1.0f / gs;
  p.local_q = (char*)local_q; p.dbg_acc = dbg_acc;
  if (push) {
    if (N != FP4AR_HIDDEN || push->nranks < 1 || push->nranks > FP4AR_MAX_RANKS || !push->call_counter) return FP4AR_ERR_ARGUMENT;
    if (M > push->cap) return FP4AR_ERR_ARGUMENT;
    p.nranks = push->nranks; p.rank = push->rank; p.cap = push->cap; p.capo = push->capo;
    p.buf_bytes = push->buffer_bytes; p.call_counter = push->call_counter; p.two_shot = two_shot ? 1 : 0;
    for (int r = 0; r < push->nranks; r++) {
      if (!push->windows[r]) return FP4AR_ERR_ARGUMENT;
      p.win[r] = (char*)push->windows[r];
    }
    // host-side bound of the farthest byte this call can touch in a window
    const size_t last = two_shot ? ((size_t)(p.nranks - 1) * p.capo + (size_t)(M - 1) / p.nranks + 1) * kRecStride
                                 : ((size_t)(p.nranks - 1) * p.cap + (size_t)M) * kRecStride;
    if (last > p.buf_bytes) return FP4AR_ERR_ARGUMENT;
  }
  p.status = gemm_status_word();
  if (!p.status) return cuda_fail();
  p.timeout_ns = 2000000000ull;
  if (stream_k) {
    StreamKSpace sp;
    if (stream_k_space(device_sm_count(), &sp)) { p.stream_k = 1; p.sk_partial = sp.partial; p.sk_flags = sp.flags; }
  }
  CUtensorMap ma, mb;
  if (!make_map(&ma, x, M, K, kBM) || !make_map(&mb, wt, N, K, pair ? bn / 2 : bn)) return FP4AR_ERR_UNSUPPORTED;
  if (pair) return launch_gemm<256, 2>(ma, mb, p, (cudaStream_t)stream);
  return bn == 192 ? launch_gemm<192, 1>(ma, mb, p, (cudaStream_t)stream) : launch_gemm<256, 1>(ma, mb, p, (cudaStream_t)stream);
}

// The schedule of one launch, computed on the host with the kernel's own iterator (for tests and tools): which shape
// a call of this size takes, and the segments of one unit as (tile, first K block, K blocks, kind) quadruples.
extern "C" int fp4ar_gemm_plan(int M, int N, int K, int sms, int* pair, int* tile_n, int* stream_k, int* units, int* tiles,
                               int unit, int* segments, int max_segments) {
  if (M < 1 || N < 256 || K < kBK || (N % 256) || (K % kBK) || sms < 2 || !pair || !tile_n || !stream_k || !units || !tiles)
    return -1;
  GemmPlan pl = plan_gemm(M, N, K, sms, /*env=*/false);
  *pair = pl.pair; *tile_n = pl.bn; *stream_k = pl.stream_k; *units = pl.units; *tiles = pl.tiles;
  if (!segments) return 0;
  if (unit < 0 || unit >= pl.units) return -1;
  SegIter it(pl.stream_k, pl.tiles, K / kBK, unit, pl.units);
  Seg sg;
  int n = 0;
  while (it.next(sg)) {
    if (n < max_segments) { segments[4 * n] = sg.tile; segments[4 * n + 1] = sg.lo; segments[4 * n + 2] = sg.count; segments[4 * n + 3] = sg.kind; }
    n++;
  }
  return n;
}

extern "C" int fp4ar_gemm_reset(void) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return cuda_fail();
  if (cudaDeviceSynchronize() != cudaSuccess) return cuda_fail();
  StatusWords* s = gemm_status_word();
  if (!s) return cuda_fail();
  if (cudaMemset(s, 0, sizeof(StatusWords)) != cudaSuccess) return cuda_fail();
  {
    std::lock_guard<std::mutex> g(g_stream_k_mu);
    const StreamKSpace& sp = g_stream_k_space[dev];
    if (sp.flags && cudaMemset(sp.flags, 0, (size_t)sp.slots * 4 * sizeof(uint32_t)) != cudaSuccess) return cuda_fail();
  }
  if (cudaDeviceSynchronize() != cudaSuccess) return cuda_fail();
  return FP4AR_OK;
}

extern "C" int fp4ar_gemm_status(fp4ar_status_words* out) {
  StatusWords* s = gemm_status_word();
  if (!s || !out) return FP4AR_ERR_ARGUMENT;
  if (cudaMemcpy(out, s, sizeof(StatusWords), cudaMemcpyDeviceToHost) != cudaSuccess) return cuda_fail();
  return FP4AR_OK;
}
