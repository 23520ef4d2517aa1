// Persistent, warp-specialised tcgen05 GEMM engine for sm_100a.
//
// One CTA per SM, (E + 2) warps where E = Epi::kEpiWarps is 4 or 8:
//   warps 0..E-1  epilogue  (warp w reads TMEM lanes 32(w%4)..32(w%4)+31 = tile rows;
//                            with E = 8, warps w and w+4 split the tile's columns, which
//                            gives every scheduler two warps to hide ALU latency with)
//   warp  E       TMA producer (one lane issues cp.async.bulk.tensor loads)
//   warp  E+1     MMA issuer   (one lane issues tcgen05.mma; also owns TMEM alloc)
//
// A tile is 128 rows x BN columns of up to kMaxSeg independent products
//   acc[s.acc] (+)= A_s[128, K_s] . B_s[BN, K_s]^T        (bf16 in, fp32 in TMEM)
// Each operand is either K-major (stored [rows][K]) or MN-major (stored
// [K][rows]); both arrive through 128-byte-swizzled TMA boxes and are consumed
// in place by the tensor core through shared-memory descriptors.  Out-of-range
// rows / K are zero-filled by TMA, so M, N, K need not be tile multiples.
//
// Accumulators live in TMEM (512 columns).  When two accumulator sets fit
// (kNumAcc * BN * 2 <= 512) the epilogue of tile i overlaps the MMAs of tile
// i+1.  The epilogue is a policy class (see the .cu files) that reads the
// accumulators with tcgen05.ld and writes whatever the fused op needs.
//
// Epilogues never store to global memory from registers (a thread owns a row,
// so a warp's store would touch 32 different lines).  Each warp stages its
// 32-row slab in 128-byte-swizzled shared memory and one lane issues a TMA
// bulk store (or reduce-add, for gradient accumulation); the hardware clips
// rows / columns outside the tensor.
//
// Every mbarrier wait is bounded.  When one runs out the CTA raises its abort
// flag, all roles leave their loops, TMEM is freed and `status` gets
// kStatusWaitTimeout; the host checks it after the launch.
#pragma once
#include <type_traits>

#include "ptx.cuh"

namespace dsb {

constexpr int kBlockM = 128;
constexpr int kBlockK = 64;   // 64 bf16 = one 128-byte swizzle row
constexpr int kMaxSeg = 3;
constexpr int kMaxOut = 8;   // output tensor maps (one per owner rank for scattered outputs)
constexpr int kTmemCols = 512;

struct GemmSeg {
  int k_tiles;  // ceil(K / 64)
  int acc;      // which accumulator this product adds into
  int a_mn;     // 1: A stored [K][M] (MN-major)
  int b_mn;     // 1: B stored [K][N] (MN-major)
};

// Fused all-gather: the A operands of a token-sharded op live in per-rank
// "full" buffers [n_ranks * rows_per_rank, cols] in symmetric memory; every
// rank has written only its own row block.  A gather warp in each CTA pulls
// the other ranks' row blocks (TMA load from the peer's buffer -> shared
// memory -> TMA store into the local buffer), then publishes a per-128-row
// ready flag; tiles that need those rows wait for the flag (bounded).  Tiles on
// this rank's own rows are scheduled first, so the transfer overlaps the math.
constexpr int kMaxGatherTensors = 3;
constexpr int kMaxRanks = 8;
struct alignas(64) GatherParams {
  CUtensorMap src[kMaxGatherTensors][kMaxRanks];  // rank j's full buffer (peer memory)
  CUtensorMap dst[kMaxGatherTensors];             // this rank's full buffer
  int cols[kMaxGatherTensors];
  int n_tensors;
  int n_ranks;        // <= 1 disables the gather
  int my_rank;
  int rows_per_rank;  // multiple of 128
  unsigned int* ready;  // [total_rows / 128] flags in local memory, compared with `epoch`
  unsigned int epoch;
  // Per-token fp32 quadruples (thresholds, 1/sigma, denominator cotangents, ...) that travel
  // with the rows: n_stats arrays of float4 [total_rows]; every rank has written its own
  // block of stat_dst[s], the gather warp copies the peers' blocks with plain 16-byte loads.
  int n_stats;
  const float4* stat_src[kMaxGatherTensors][kMaxRanks];
  float4* stat_dst[kMaxGatherTensors];
  // Raw views of the same buffers for the register-copy gather (kGather == 2): base
  // pointers and the row stride in 16-byte units.
  const uint4* src_ptr[kMaxGatherTensors][kMaxRanks];
  uint4* dst_ptr[kMaxGatherTensors];
  long long ld16[kMaxGatherTensors];
};
// Gather modes of the engine kernel (template parameter kGather):
//   0  none
//   1  TMA load from the peer -> a ring of four 8 KB bounce buffers in shared memory -> TMA
//      store, three loads in flight.  Highest copy rate per CTA, but the 32 KB cost the
//      operand ring one stage.
//   2  two warps copy through registers (16-byte loads from the peer, 16-byte stores into
//      the local buffer, eight in flight per lane): no shared memory, so the ring keeps
//      all its stages; the copy rate is lower and suits kernels that run long enough to
//      hide it (large unit shards).
constexpr int kGatherNone = 0, kGatherBounce = 1, kGatherRegs = 2;

template <class EpiParams>
struct alignas(64) GemmParams {
  CUtensorMap tma_a[kMaxSeg];
  CUtensorMap tma_b[kMaxSeg];
  CUtensorMap tma_out[kMaxOut];  // epilogue outputs: box = 128 bytes x 32 rows, 128B swizzle
  GemmSeg seg[kMaxSeg];
  int n_seg;
  int M, N;
  int m_tiles, n_tiles;
  int n_fastest;  // tile raster: 1 = consecutive tiles walk N first
  int m_rot;      // tile rows are visited starting from this m-tile (own rows first)
  int m_first;    // > 0 with an M-fastest raster: the first m_first (rotated) tile rows - this
                  // rank's own rows - are swept completely before the others, so a fused
                  // gather has that long to land the peers' rows
  int k_splits;   // > 1: the K range of segment 0 is cut into this many tiles that all
                  // reduce-add into the same output (accumulating fp32 epilogues only)
  GatherParams gather;
  int* status;    // device word, set non-zero on failure
  EpiParams epi;
};

constexpr int kOutBufBytes = 4096;  // one staged slab: 32 rows x 128 bytes

constexpr int kGatherPieceBytes = 64 * 64 * 2;    // 64 rows x 64 bf16
constexpr int kGatherSlots = 4;                   // bounce buffers of the ring
template <int BN, int kOutBufsPerWarp, int kEpiWarps = 4, int kGather = 0>
struct EngineSmem {
  static constexpr int kABytes = kBlockM * kBlockK * 2;  // 16 KB
  static constexpr int kBBytes = BN * kBlockK * 2;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kGatherBytes = kGather == kGatherBounce ? kGatherSlots * kGatherPieceBytes : 0;
  static constexpr int kOutBytes = kEpiWarps * kOutBufsPerWarp * kOutBufBytes + kGatherBytes;
  static constexpr int kMaxSmem = 227 * 1024;
  static constexpr int kBudget = kMaxSmem - kOutBytes - 1024 /*align slack*/ - 512 /*barriers*/;
  static constexpr int kStages = (kBudget / kStageBytes) > 8 ? 8 : (kBudget / kStageBytes);
  static constexpr int kTileBytes = kStages * kStageBytes;
  static constexpr int kTotalBytes = kTileBytes + kOutBytes + 1024 + 512;
  static_assert(kStages >= 2, "not enough shared memory for a pipeline");
};

// Per-warp staging of epilogue output slabs (32 rows x 128 bytes each).
// Thread `lane` owns row `lane`; 16-byte chunk c of its row lives at
// lane*128 + ((c ^ (lane & 7)) << 4), the layout a 128B-swizzled TMA box reads.
struct WarpStager {
  uint32_t base;  // shared address of this warp's first buffer
  int lane;
  __device__ __forceinline__ uint32_t buf(int i) const { return base + i * kOutBufBytes; }
  // Block until at most `kPending` of this warp's bulk stores still read smem.
  template <int kPending>
  __device__ __forceinline__ void wait_free() const {
    if (lane == 0) bulk_wait_read<kPending>();
    __syncwarp();
  }
  __device__ __forceinline__ void put(uint32_t buf_addr, int chunk, uint32_t a, uint32_t b,
                                      uint32_t c, uint32_t d) const {
    st_shared_v4(buf_addr + lane * 128 + ((chunk ^ (lane & 7)) << 4), a, b, c, d);
  }
  // Make the staged slab visible to the async proxy and store it at
  // (c0, r0).  Always commits a group so waits can count slabs.
  __device__ __forceinline__ void flush(const CUtensorMap* map, uint32_t buf_addr, int c0, int r0,
                                        bool reduce_add, bool issue) const {
    publish();
    store(map, buf_addr, c0, r0, reduce_add, issue);
  }
  // The two halves of flush(), for staging several slabs behind one fence.
  __device__ __forceinline__ void publish() const {
    fence_proxy_async_smem();
    __syncwarp();
  }
  __device__ __forceinline__ void store(const CUtensorMap* map, uint32_t buf_addr, int c0, int r0,
                                        bool reduce_add, bool issue) const {
    if (lane == 0) {
      if (issue) {
        if (reduce_add) tma_reduce_add_2d(map, buf_addr, c0, r0);
        else tma_store_2d(map, buf_addr, c0, r0);
      }
      bulk_commit();
    }
  }
};

// Accumulator hand-off between the MMA issuer and the epilogue warps.  Every
// accumulator `a` of a tile has Epi::acc_bufs(a) TMEM buffers (1 or 2) and its
// own full/empty barrier pair, so a policy can read (and free) one accumulator
// while the tensor core still works on another one of the same tile, and an
// accumulator with two buffers lets the next tile start while this tile's
// epilogue runs.  Per tile every epilogue warp must wait() and release() each
// accumulator exactly once (skip() does both without reading).
template <int BN, class Epi, int kCtas>
struct AccCtl {
  uint64_t* full;    // [kNumAcc][2]
  uint64_t* empty;   // [kNumAcc][2]
  uint32_t tmem_lanes;  // TMEM base address with this warp's lane offset
  int it;               // tiles processed so far by this CTA
  int lane;
  volatile int* abort_flag;
  bool ok;

  __device__ __forceinline__ static constexpr int col_off(int a) {
    int c = 0;
    for (int b = 0; b < a; ++b) c += Epi::acc_bufs(b) * BN;
    return c;
  }
  // Wait until accumulator `a` of this tile is complete; returns its TMEM address.
  __device__ __forceinline__ uint32_t wait(int a) {
    const int nb = Epi::acc_bufs(a), j = it % nb;
    const uint32_t use = static_cast<uint32_t>(it / nb);
    if (ok && !mbar_wait(&full[a * 2 + j], use & 1, abort_flag)) ok = false;
    tc_fence_after();
    return tmem_lanes + col_off(a) + j * BN;
  }
  // This warp is done reading accumulator `a` of this tile.
  __device__ __forceinline__ void release(int a) {
    const int nb = Epi::acc_bufs(a), j = it % nb;
    tc_fence_before();
    __syncwarp();
    if (lane == 0) {
      if (kCtas == 2) mbar_arrive_cluster(mapa_shared(smem_u32(&empty[a * 2 + j]), 0));
      else mbar_arrive(&empty[a * 2 + j]);
    }
  }
  __device__ __forceinline__ void skip() {
#pragma unroll
    for (int a = 0; a < Epi::kNumAcc; ++a) { wait(a); release(a); }
  }
};

// Epilogue policy contract:
//   static constexpr int kNumAcc;
//   struct Params;
//   static constexpr int kNumOut;    // output tensor maps used
//   static constexpr int kOutBufs;   // staging buffers per epilogue warp
//   static constexpr int kEpiWarps;  // 4 or 8
//   static constexpr int acc_bufs(int a);   // TMEM buffers of accumulator a (1 or 2)
//   __device__ static void run(const Params&, const CUtensorMap* out_maps, WarpStager&,
//                              AccCtl&, int m0, int n0, int M, int N, int warp, int lane);
// `warp` is the epilogue warp index (0..kEpiWarps-1); its rows are
// m0 + 32*(warp%4) + lane and, with 8 warps, its columns the (warp/4)-th half.

// Threads per CTA.  With 8 epilogue warps the CTA is padded to three full warpgroups
// (12 warps; warps 8.. are TMA, MMA, gather and idle) so that registers can be moved
// between warpgroups: each SM sub-partition holds warps w, w+4 and w+8 and the kernel is
// launched with 168 registers per thread.  The helper warpgroup gives most of its share
// back (setmaxnreg.dec) and the two epilogue warpgroups, which keep 128 packed accumulator
// values per thread, take it (setmaxnreg.inc).
template <class Epi, int kGather>
constexpr int engine_threads() {
  return Epi::kEpiWarps == 8 ? 384 : (Epi::kEpiWarps + 2 + (kGather ? 1 : 0)) * 32;
}
constexpr int kHelperRegs = 88;     // TMA / MMA / gather warps after setmaxnreg.dec
constexpr int kEpilogueRegs = 208;  // epilogue warps after setmaxnreg.inc
// Registers only move inside what the CTA was launched with: 168 per thread, i.e. 3 x 168 =
// 504 per lane of a sub-partition.  A split that asks for more makes setmaxnreg.inc wait for
// registers that never come, and that wait has no time limit.
static_assert(2 * kEpilogueRegs + kHelperRegs <= 3 * 168, "register split exceeds the launch allocation");
static_assert(kEpilogueRegs % 8 == 0 && kHelperRegs % 8 == 0, "setmaxnreg takes multiples of 8");

// (m-tile, n-tile) of the t2-th output tile of the raster described by the launch parameters.
template <class P>
__device__ __forceinline__ void tile_coords(const P& p, int t2, int& mt, int& nt) {
  if (p.n_fastest) {
    mt = t2 / p.n_tiles;
    nt = t2 - mt * p.n_tiles;
  } else if (p.m_first > 0 && p.m_first < p.m_tiles) {
    const int first = p.m_first * p.n_tiles;
    if (t2 < first) {
      nt = t2 / p.m_first;
      mt = t2 - nt * p.m_first;
    } else {
      const int rest = p.m_tiles - p.m_first, t3 = t2 - first;
      nt = t3 / rest;
      mt = p.m_first + (t3 - nt * rest);
    }
  } else {
    nt = t2 / p.m_tiles;
    mt = t2 - nt * p.m_tiles;
  }
  mt += p.m_rot;
  if (mt >= p.m_tiles) mt -= p.m_tiles;
}

template <int BN, class Epi, int kCtas, int kGather = 0>
__global__ void __launch_bounds__(engine_threads<Epi, kGather>(), 1)
gemm_engine_kernel(const __grid_constant__ GemmParams<typename Epi::Params> p) {
  // kCtas == 2: the CTA pair of a 2-CTA cluster shares a 256-row tile.  Each CTA
  // stages its own 128 rows of A and BN/2 rows of B; the leader CTA (cluster
  // rank 0) issues tcgen05.mma.cta_group::2 for both.  All TMA loads count
  // their bytes on the leader's `full` barrier; MMA completion is multicast to
  // both CTAs' `empty` / `acc_full` barriers; both CTAs' epilogue warps arrive
  // on the leader's `acc_empty`.
  static_assert(kCtas == 1 || kCtas == 2, "1 or 2 CTAs per tile");
  constexpr int kBRows = BN / kCtas;  // rows of B this CTA stages
  using Smem = EngineSmem<kBRows, Epi::kOutBufs, Epi::kEpiWarps, kGather>;
  constexpr int kEpiWarps = Epi::kEpiWarps;
  constexpr int kTmaWarp = kEpiWarps, kMmaWarp = kEpiWarps + 1, kGatherWarp = kEpiWarps + 2;
  static_assert(kEpiWarps == 4 || kEpiWarps == 8, "4 or 8 epilogue warps");
  constexpr int kNumAcc = Epi::kNumAcc;
  using Ctl = AccCtl<BN, Epi, kCtas>;
  static_assert(Ctl::col_off(kNumAcc) <= kTmemCols, "accumulators exceed TMEM");
  constexpr int kStages = Smem::kStages;
  constexpr int kTileM = kBlockM * kCtas;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* out_stage = smem + Smem::kTileBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(out_stage + Smem::kOutBytes);
  uint64_t* full_bar = bars;                       // [kStages]
  uint64_t* empty_bar = bars + kStages;            // [kStages]
  uint64_t* acc_full = bars + 2 * kStages;         // [kMaxSeg][2]
  uint64_t* acc_empty = bars + 2 * kStages + 6;    // [kMaxSeg][2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * kStages + 12);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  uint64_t* gather_bar = bars + 2 * kStages + 14;  // [kGatherSlots]
  uint8_t* gather_buf = out_stage + kEpiWarps * Epi::kOutBufs * kOutBufBytes;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = (kCtas == 2) ? cluster_ctarank() : 0u;
  const bool leader = rank == 0;
  const int tile_stride = gridDim.x / kCtas;
  const int first_tile = blockIdx.x / kCtas;

  if (threadIdx.x == 0) {
    for (int i = 0; i < kStages; ++i) {
      mbar_init(&full_bar[i], 1);
      mbar_init(&empty_bar[i], 1);
    }
    for (int i = 0; i < 2 * kMaxSeg; ++i) {
      mbar_init(&acc_full[i], 1);
      mbar_init(&acc_empty[i], kCtas * kEpiWarps);   // one elected arrive per epilogue warp
    }
    if (kGather == kGatherBounce) {
      for (int i = 0; i < kGatherSlots; ++i) mbar_init(&gather_bar[i], 1);
    }
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == kTmaWarp && lane == 0) {
    for (int s = 0; s < p.n_seg; ++s) {
      tma_prefetch_desc(&p.tma_a[s]);
      tma_prefetch_desc(&p.tma_b[s]);
    }
  }
  if (warp == 0 && lane == 0) {
    for (int s = 0; s < Epi::kNumOut; ++s) tma_prefetch_desc(&p.tma_out[s]);
  }
  if (warp == kMmaWarp) {
    if (kCtas == 2) { tmem_alloc_pair(tmem_slot, kTmemCols); tmem_relinquish_pair(); }
    else { tmem_alloc(tmem_slot, kTmemCols); tmem_relinquish(); }
  }
  tc_fence_before();
  __syncthreads();
  if (kCtas == 2) cluster_sync_all();   // peer barriers are initialised before anyone signals them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const int mn_tiles = p.m_tiles * p.n_tiles;
  const int k_splits = p.k_splits > 1 ? p.k_splits : 1;
  const int total_tiles = mn_tiles * k_splits;
  // k-tiles of segment 0 handled by one split (the last split may get fewer)
  const int kt_per_split = (p.seg[0].k_tiles + k_splits - 1) / k_splits;

  if (warp >= kEpiWarps) {
  // ======================================================= helper warpgroup
  if constexpr (kEpiWarps == 8)
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kHelperRegs));
  if (warp == kTmaWarp) {
    // ------------------------------------------------------------ producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      constexpr int kSeenWords = 32;      // 1024 row blocks of 128 rows
      uint32_t seen[kSeenWords];          // gathered row blocks whose flag this CTA has seen
      if (kGather) {
#pragma unroll
        for (int i = 0; i < kSeenWords; ++i) seen[i] = 0u;
      }
      for (int tile = first_tile; tile < total_tiles && ok; tile += tile_stride) {
        const int ks = tile / mn_tiles, t2 = tile - ks * mn_tiles;
        int mt, nt;
        tile_coords(p, t2, mt, nt);
        const int m0 = mt * kTileM + static_cast<int>(rank) * kBlockM;
        const int n0 = nt * BN + static_cast<int>(rank) * kBRows;
        if (kGather && p.gather.n_ranks > 1 && m0 < p.M &&
            m0 / p.gather.rows_per_rank != p.gather.my_rank) {
          // rows of another rank: wait until the gather warps have landed them here; a block
          // seen once needs no second system-scope acquire
          const int blk = m0 / 128;
          const bool known = blk < 32 * kSeenWords && ((seen[blk >> 5] >> (blk & 31)) & 1u);
          if (!known) {
            if (!flag_wait_ge(p.gather.ready + blk, p.gather.epoch, abort_flag)) { ok = false; break; }
            fence_proxy_async_global();
            if (blk < 32 * kSeenWords) seen[blk >> 5] |= 1u << (blk & 31);
          }
        }
        for (int s = 0; s < p.n_seg && ok; ++s) {
          const GemmSeg sg = p.seg[s];
          const int kt_lo = k_splits > 1 ? ks * kt_per_split : 0;
          const int kt_hi = k_splits > 1 ? min(sg.k_tiles, kt_lo + kt_per_split) : sg.k_tiles;
          for (int kt = kt_lo; kt < kt_hi; ++kt) {
            if (!mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag)) { ok = false; break; }
            uint8_t* sa = smem + stage * Smem::kStageBytes;
            uint8_t* sb = sa + Smem::kABytes;
            const int k0 = kt * kBlockK;
            if (kCtas == 1) {
              mbar_expect_tx(&full_bar[stage], Smem::kStageBytes);
              if (sg.a_mn) {
                tma_load_2d(sa, &p.tma_a[s], &full_bar[stage], m0, k0);
                tma_load_2d(sa + 8192, &p.tma_a[s], &full_bar[stage], m0 + 64, k0);
              } else {
                tma_load_2d(sa, &p.tma_a[s], &full_bar[stage], k0, m0);
              }
              if (sg.b_mn) {
#pragma unroll
                for (int j = 0; j < kBRows / 64; ++j)
                  tma_load_2d(sb + j * 8192, &p.tma_b[s], &full_bar[stage], n0 + 64 * j, k0);
              } else {
                tma_load_2d(sb, &p.tma_b[s], &full_bar[stage], k0, n0);
              }
            } else {
              // bytes of both CTAs are counted on the leader's barrier
              if (leader) mbar_expect_tx(&full_bar[stage], 2 * Smem::kStageBytes);
              const uint32_t fb = mapa_shared(smem_u32(&full_bar[stage]), 0);
              if (sg.a_mn) {
                tma_load_2d_pair(sa, &p.tma_a[s], fb, m0, k0);
                tma_load_2d_pair(sa + 8192, &p.tma_a[s], fb, m0 + 64, k0);
              } else {
                tma_load_2d_pair(sa, &p.tma_a[s], fb, k0, m0);
              }
              if (sg.b_mn) {
#pragma unroll
                for (int j = 0; j < kBRows / 64; ++j)
                  tma_load_2d_pair(sb + j * 8192, &p.tma_b[s], fb, n0 + 64 * j, k0);
              } else {
                tma_load_2d_pair(sb, &p.tma_b[s], fb, k0, n0);
              }
            }
            if (++stage == kStages) { stage = 0; phase ^= 1; }
          }
        }
      }
    }
  } else if (warp == kMmaWarp) {
    // ---------------------------------------------------------- MMA issuer
    // One thread feeds the tensor pipe, which queues only about one
    // instruction ahead, so everything between two tcgen05.mma must be cheap:
    // descriptor increments are compile-time constants (the loop body is
    // instantiated per operand layout) and the barrier wait has a one-
    // instruction fast path.
    if (lane == 0 && leader) {
      int stage = 0;
      uint32_t phase = 0;
      int it = 0;
      bool ok = true;
      const uint32_t smem_base = smem_u32(smem);
      const int n_seg = p.n_seg;
      auto issue_seg = [&](auto a_mn_c, auto b_mn_c, const int k_tiles, const uint32_t d_tmem,
                           uint32_t accum) {
        constexpr bool kAmn = decltype(a_mn_c)::value, kBmn = decltype(b_mn_c)::value;
        constexpr uint32_t kAInc = (kAmn ? 2048u : 32u) >> 4, kBInc = (kBmn ? 2048u : 32u) >> 4;
        const uint32_t idesc = umma_idesc_bf16(kTileM, BN, kAmn, kBmn);
        const uint64_t a_base = umma_desc(smem_base, kAmn ? 8192u : 16u, 1024);
        const uint64_t b_base = umma_desc(smem_base + Smem::kABytes, kBmn ? 8192u : 16u, 1024);
#pragma unroll 1
        for (int kt = 0; kt < k_tiles; ++kt) {
          if (!mbar_try_wait(&full_bar[stage], phase) &&
              !mbar_wait(&full_bar[stage], phase, abort_flag)) { ok = false; return; }
          tc_fence_after();
          const uint64_t so = static_cast<uint64_t>(static_cast<uint32_t>(stage) *
                                                    (Smem::kStageBytes >> 4));
          const uint64_t ad = a_base + so, bd = b_base + so;
#pragma unroll
          for (int kk = 0; kk < kBlockK / 16; ++kk) {
            if (kCtas == 2) mma_bf16_ss_pair(d_tmem, ad + kk * kAInc, bd + kk * kBInc, idesc, accum);
            else mma_bf16_ss(d_tmem, ad + kk * kAInc, bd + kk * kBInc, idesc, accum);
            accum = 1u;
          }
          // frees the smem stage (in both CTAs) when the MMAs retire
          if (kCtas == 2) mma_commit_pair(&empty_bar[stage]);
          else mma_commit(&empty_bar[stage]);
          if (++stage == kStages) { stage = 0; phase ^= 1; }
        }
      };
      using T_ = std::true_type;
      using F_ = std::false_type;
      for (int tile = first_tile; tile < total_tiles && ok; tile += tile_stride, ++it) {
        for (int s = 0; s < n_seg && ok; ++s) {
          const GemmSeg sg = p.seg[s];
          // one segment per accumulator: wait for its buffer, fill it, publish it
          const int nb = Epi::acc_bufs(sg.acc), j = it % nb;
          const uint32_t use = static_cast<uint32_t>(it / nb);
          if (!mbar_wait(&acc_empty[sg.acc * 2 + j], (use & 1) ^ 1, abort_flag)) { ok = false; break; }
          tc_fence_after();
          const uint32_t d_tmem = tmem_base + Ctl::col_off(sg.acc) + j * BN;
          int nk = sg.k_tiles;
          if (k_splits > 1) {
            const int ks = tile / mn_tiles;
            nk = min(sg.k_tiles, (ks + 1) * kt_per_split) - ks * kt_per_split;
            if (nk < 0) nk = 0;
          }
          if (!sg.a_mn && !sg.b_mn) issue_seg(F_{}, F_{}, nk, d_tmem, 0u);
          else if (!sg.a_mn && sg.b_mn) issue_seg(F_{}, T_{}, nk, d_tmem, 0u);
          else if (sg.a_mn && !sg.b_mn) issue_seg(T_{}, F_{}, nk, d_tmem, 0u);
          else issue_seg(T_{}, T_{}, nk, d_tmem, 0u);
          if (ok) {
            if (kCtas == 2) mma_commit_pair(&acc_full[sg.acc * 2 + j]);
            else mma_commit(&acc_full[sg.acc * 2 + j]);
          }
        }
      }
    }
  } else if (kGather == kGatherRegs &&
             (warp == kGatherWarp || (kEpiWarps == 8 && warp == kGatherWarp + 1))) {
    // ------------------------------------------- gather through registers
    const GatherParams& g = p.gather;
    if (g.n_ranks > 1) {
      constexpr int kGW = kEpiWarps == 8 ? 2 : 1;          // gather warps per CTA
      const int cpr = g.rows_per_rank / 128;               // 128-row chunks per rank
      const int remote = (g.n_ranks - 1) * cpr;
      for (int rc = blockIdx.x * kGW + (warp - kGatherWarp); rc < remote; rc += gridDim.x * kGW) {
        const int owner = (g.my_rank + 1 + rc / cpr) % g.n_ranks;
        const int grow = owner * g.rows_per_rank + (rc % cpr) * 128;
        for (int sidx = 0; sidx < g.n_stats; ++sidx) {
          const float4* src = g.stat_src[sidx][owner] + grow;
          float4* dst = g.stat_dst[sidx] + grow;
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            float4 v;
            asm volatile("ld.global.cv.v4.f32 {%0,%1,%2,%3}, [%4];"
                         : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
                         : "l"(src + lane + 32 * k)
                         : "memory");
            dst[lane + 32 * k] = v;
          }
        }
        for (int t = 0; t < g.n_tensors; ++t) {
          const int vpr = g.cols[t] >> 3;                  // 16-byte vectors per row
          const int total = 128 * vpr;                     // a multiple of 256 (cols % 64 == 0)
          const uint4* src = g.src_ptr[t][owner] + static_cast<size_t>(grow) * g.ld16[t];
          uint4* dst = g.dst_ptr[t] + static_cast<size_t>(grow) * g.ld16[t];
          for (int v0 = 0; v0 < total; v0 += 256) {
            uint4 q[8];
            size_t off[8];
#pragma unroll
            for (int k = 0; k < 8; ++k) {
              const int v = v0 + lane + 32 * k;
              off[k] = static_cast<size_t>(v / vpr) * g.ld16[t] + (v % vpr);
              asm volatile("ld.global.cv.v4.u32 {%0,%1,%2,%3}, [%4];"
                           : "=r"(q[k].x), "=r"(q[k].y), "=r"(q[k].z), "=r"(q[k].w)
                           : "l"(src + off[k])
                           : "memory");
            }
#pragma unroll
            for (int k = 0; k < 8; ++k) dst[off[k]] = q[k];
          }
        }
        __threadfence();             // every lane's stores are visible before the flag
        __syncwarp();
        if (lane == 0) flag_store_release(g.ready + grow / 128, g.epoch);
      }
    }
  } else if (kGather == kGatherBounce && warp == kGatherWarp) {
    // ------------------------------- gather through shared-memory bounce buffers
    // A ring of kGatherSlots pieces (64 rows x 64 columns): up to kGatherSlots - 1 loads
    // from the peer are in flight while landed pieces are stored to local memory.
    const GatherParams& g = p.gather;
    if (g.n_ranks > 1) {
      const int cpr = g.rows_per_rank / 128;               // 128-row chunks per rank
      const int remote = (g.n_ranks - 1) * cpr;
      int strips = 0;                                      // 64-column strips over all tensors
      for (int t = 0; t < g.n_tensors; ++t) strips += g.cols[t] >> 6;
      const int ppc = 2 * strips;                          // pieces per chunk
      const int my_chunks = (remote > static_cast<int>(blockIdx.x))
                                ? (remote - 1 - static_cast<int>(blockIdx.x)) / static_cast<int>(gridDim.x) + 1
                                : 0;
      const int total = my_chunks * ppc;
      // piece q -> (owner row block, tensor, column, row half)
      auto locate = [&](int q, int& t, int& c0, int& grow, int& owner) {
        const int rc = static_cast<int>(blockIdx.x) + (q / ppc) * static_cast<int>(gridDim.x);
        owner = (g.my_rank + 1 + rc / cpr) % g.n_ranks;   // nearer ranks first, a different peer per rank
        grow = owner * g.rows_per_rank + (rc % cpr) * 128;
        int w = q % ppc;
        const int half = w & 1;
        w >>= 1;
        t = 0;
        while (w >= (g.cols[t] >> 6)) { w -= g.cols[t] >> 6; ++t; }
        c0 = w << 6;
        grow += 64 * half;
      };
      auto issue_load = [&](int q) {
        int t, c0, grow, owner;
        locate(q, t, c0, grow, owner);
        const int slot = q % kGatherSlots;
        mbar_expect_tx(&gather_bar[slot], kGatherPieceBytes);
        tma_load_2d(gather_buf + slot * kGatherPieceBytes, &g.src[t][owner], &gather_bar[slot], c0, grow);
      };
      bool ok = true;
      if (lane == 0)
        for (int q = 0; q < kGatherSlots - 1 && q < total; ++q) issue_load(q);
      for (int done = 0; done < total && ok; ++done) {
        int t, c0, grow, owner;
        locate(done, t, c0, grow, owner);
        if (lane == 0) {
          const int slot = done % kGatherSlots;
          ok = mbar_wait(&gather_bar[slot], static_cast<uint32_t>(done / kGatherSlots) & 1u, abort_flag);
          if (ok) {
            tma_store_2d(&g.dst[t], smem_u32(gather_buf + slot * kGatherPieceBytes), c0, grow);
            bulk_commit();
            const int nxt = done + kGatherSlots - 1;
            if (nxt < total) {
              bulk_wait_read<1>();   // the store that last used the next load's slot has read it
              issue_load(nxt);
            }
          }
        }
        ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
        if (!ok) break;
        if (done % ppc == ppc - 1) {
          // last piece of a chunk: copy its per-token statistics (all lanes), wait for the
          // chunk's stores, publish the block
          const int crow = grow - 64;                      // the last piece is a second half
          for (int sidx = 0; sidx < g.n_stats; ++sidx) {
            const float4* src = g.stat_src[sidx][owner] + crow;
            float4* dst = g.stat_dst[sidx] + crow;
#pragma unroll
            for (int k = 0; k < 4; ++k) {
              float4 v;
              asm volatile("ld.global.cv.v4.f32 {%0,%1,%2,%3}, [%4];"
                           : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
                           : "l"(src + lane + 32 * k)
                           : "memory");
              dst[lane + 32 * k] = v;
            }
          }
          if (lane == 0) bulk_wait<0>();                   // the chunk's rows are in local memory
          __threadfence();
          __syncwarp();
          if (lane == 0) flag_store_release(g.ready + crow / 128, g.epoch);
        }
      }
      if (lane == 0) bulk_wait<0>();
    }
  }
  } else {
    // ------------------------------------------------------------ epilogue
    if constexpr (kEpiWarps == 8)
      asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kEpilogueRegs));
    int it = 0;
    bool ok = true;
    WarpStager stager{smem_u32(out_stage + warp * Epi::kOutBufs * kOutBufBytes), lane};
    for (int tile = first_tile; tile < total_tiles && ok; tile += tile_stride, ++it) {
      const int t2 = tile % mn_tiles;
      int mt, nt;
      tile_coords(p, t2, mt, nt);
      Ctl ctl{acc_full, acc_empty, tmem_base + (static_cast<uint32_t>((warp & 3) * 32) << 16), it,
              lane, abort_flag, true};
      Epi::template run<BN>(p.epi, p.tma_out, stager, ctl,
                            mt * kTileM + static_cast<int>(rank) * kBlockM, nt * BN, p.M, p.N, warp,
                            lane);
      ok = ctl.ok;
    }
    if (lane == 0) bulk_wait<0>();  // all of this warp's bulk stores have landed
  }

  // ---------------------------------------------------------------- teardown
  __syncwarp();
  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    if (threadIdx.x == 0 && p.status != nullptr) atomicExch(p.status, kStatusWaitTimeout);
    // give copies / MMAs that may still be in flight time to land before the
    // shared memory and TMEM they target are released
    const long long t0 = clock64();
    while (clock64() - t0 < 2000000LL) { }
    __syncthreads();
  }
  if (kCtas == 2) cluster_sync_all();   // neither CTA leaves while its peer may still signal it
  if (warp == kMmaWarp) {
    tc_fence_after();
    if (kCtas == 2) tmem_dealloc_pair(tmem_base, kTmemCols);
    else tmem_dealloc(tmem_base, kTmemCols);
  }
}

}  // namespace dsb
