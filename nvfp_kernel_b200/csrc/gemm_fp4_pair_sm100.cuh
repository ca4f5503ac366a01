// Block-scaled FP4 GEMM on CTA pairs (tcgen05 cta_group::2): one cluster of two CTAs on a
// TPC computes a 256 x 256 output tile.  Included by gemm_fp4_sm100.cu inside namespace
// nvfp::<anonymous>; uses its GemmParams, store_row_chunk and tensor-map helpers.
//
// Why pairs: per 64 elements of K a single CTA computing 128 x 256 must bring 128 + 256 operand
// rows through L2 and its own shared memory; a pair computing 256 x 256 brings 128 + 128 rows
// per CTA for twice the flops, because the tensor cores of the two SMs exchange their halves of B.
// The reference's kernel (CUTLASS Sm120, cluster 1x1x1, kernel/nvfp4_scaled_mm_sm120_kernels.cu:52-70)
// has no such mode.
//
// Roles per CTA (192 threads):
//   warp 0   producer: TMA loads of its 128 rows of A, its 128 rows of B, its 128 rows of A
//            scales and all 256 rows of B scales into its own shared memory; completion is
//            reported to the LEADER's (cluster rank 0) "full" barrier
//   warp 1   leader only: issuer of tcgen05.cp / tcgen05.mma for both CTAs
//   warps 2-5 epilogue of this CTA's 128 accumulator rows
// Every load is issued by the CTA that consumes it (no cluster-wide broadcast loads).
#pragma once

constexpr int kPairBM = 256;
constexpr int kPairBN = 256;
// Tile numbering (pair_tile_coords): the rows of A that one band of tile rows covers should stay in L2 while all of B
// streams past them once per band; this many bytes of A (values and scales) per band at most.
constexpr int64_t kPairBandBytes = 40ll << 20;

template <bool MX>
struct PairCfg {
  static constexpr int kChunksPerStage = MX ? 2 : 4;
  static constexpr int kMmasPerChunk = MX ? 2 : 1;
  static constexpr uint32_t kABytes = 128 * kStageKBytes;                    // this CTA's rows of A
  static constexpr uint32_t kBBytes = 128 * kStageKBytes;                    // this CTA's half of B
  static constexpr uint32_t kSfaBytes = kChunksPerStage * 512;
  static constexpr uint32_t kSfbBytes = 2 * kChunksPerStage * 512;           // both 128-row tiles of B scales
  static constexpr uint32_t kStageBytes = kABytes + kBBytes + kSfaBytes + kSfbBytes;
  // epilogue staging: per epilogue warp two buffers of 32 rows x 128 bytes (128-byte swizzle)
  static constexpr uint32_t kStoreBufBytes = 32 * 128;
  static constexpr uint32_t kStagingBytes = 4 * 2 * kStoreBufBytes;
  // NVFP4-gather epilogue: the scale bytes of one 128-row x 256-column tile (four 512-byte chunks), staged by the four
  // epilogue warps together
  static constexpr uint32_t kSfStagingBytes = 4 * 512;
  static constexpr int kStages = (kSmemLimit - 2048 - kStagingBytes - kSfStagingBytes) / kStageBytes;
  static constexpr uint32_t kSmemBytes = kStages * kStageBytes + kStagingBytes + kSfStagingBytes + 2048;
  // Tensor-memory columns.  Two 256-column accumulators do not fit beside the scale columns, so they
  // OVERLAP: even tiles accumulate in [0,256), odd tiles in [208,464), scales live in [464,512).  The
  // epilogue drains the shared columns [208,256) first and releases the accumulator barrier right
  // after, so the next tile's MMAs start while the other 208 columns are still being stored.
  static constexpr uint32_t kSfaCols = 4 * kChunksPerStage;
  static constexpr uint32_t kSfbCols = 8 * kChunksPerStage;
  static constexpr uint32_t kSfColBase = kTmemCols - 48;
  static constexpr uint32_t kOddAccCol = kSfColBase - kPairBN;          // 208
  static constexpr int kEarlyChunks = 2;   // 32-column chunks that cover the shared columns
  static_assert(kSfaCols + kSfbCols <= 48, "scale columns");
  static_assert(kOddAccCol % 16 == 0 && kOddAccCol + 32 * kEarlyChunks >= kPairBN, "overlap covered by the early chunks");
};

// Output tensor maps: entry 0 is this GPU's [M, N] output; further entries are the same-shaped
// destinations in peer GPUs' memory (column-parallel layers write their slab straight into every
// peer's gathered buffer instead of running an all-gather afterwards).
constexpr int kMaxOutputs = 8;
struct OutMaps {
  CUtensorMap map[kMaxOutputs];
};
// How the epilogue uses the output maps:
//   kOutStoreAll    every tile is stored to all n_out destinations (1 = plain GEMM, >1 = fused gather)
//   kOutScatterAdd  row-parallel (K-split) layers: destination r owns rows [r*rows_per_owner, ...) of the
//                   result; each 32-row block of this rank's fp32 partial product is ADDED (TMA reduce)
//                   into its owner's buffer -- the reduce-scatter fused into the epilogue
//   kOutFused       the epilogue applies the gated activation (p.act) and / or quantizes to NVFP4 (p.out_gs) and
//                   stores from registers (finish_row_chunk); no output maps
//   kOutFp4Gather   the tile is quantized to NVFP4 in the epilogue (p.out_gs) and its packed bytes and scale bytes are
//                   stored to all n_out destinations: the column-parallel gather of the NEXT layer's activation
//                   operand, 0.5625 bytes per element over NVLink instead of 2
constexpr int kOutStoreAll = 0, kOutScatterAdd = 1, kOutFused = 2, kOutFp4Gather = 3;

// Scale destinations of kOutFp4Gather, in the order of the output maps: base of each destination's swizzled scale
// tensor ([rowTile][kTile][512 bytes] of the GATHERED [m, n_total] matrix), and where this rank's columns sit in it.
struct GatherFp4 {
  uint8_t* sf[kMaxOutputs];
  int k_tiles_total;    // 64-column scale tiles per row tile of the gathered matrix
  int k_tile0;          // first scale tile of this rank's slab
  int k_tiles_slab;     // scale tiles of this rank's slab (n / 64)
};

// Synchronisation of the ranks of a tensor-parallel layer INSIDE the GEMM kernel, through flag words in peer-visible
// memory (plain system-scope stores and loads over NVLink; no collective, no extra launch).  Every rank owns a block of
// kPeerFlagWords uint32, zeroed once:
//   [0, 8)   ready[r]   rank r has reached call number ready[r]: nobody on r reads r's destination buffer any more
//   [8, 16)  done[r]    everything rank r writes into THIS rank's buffer in call number done[r] has arrived
//   [16]     epilogue warps of this GPU that have finished the current call (reset by the last one)
//   [17]     number of completed calls (the sequence number; kept on the device so that a replayed launch still counts)
// At its start a kernel announces ready on every peer; an epilogue warp waits for a peer's ready before its first
// store to that peer; the last epilogue warp to finish announces done on every peer and waits for every peer's done,
// so the gathered (or reduced) result is complete when the kernel ends.  Every wait is bounded: on expiry the warp
// records kErrPeerWait in the device status word and goes on -- without its remote stores, if the wait was for ready.
constexpr int kPeerFlagWords = 32;
constexpr uint32_t kErrPeerWait = 32u;
struct PeerSync {
  uint32_t* flags[kMaxOutputs];   // rank r's flag block (peer-mapped for r != rank)
  int world;                      // 0: the caller synchronises the ranks around the call
  int rank;
  uint64_t limit_ns;              // bound of each wait
};

#ifdef NVFP_PAIR_TRACE
// Instrumented build (python -m nvfp_kernel_b200.build --trace): where do the roles of a CTA pair spend their clocks?
// Per cluster: [0] issuer, clocks from its first to its last instruction  [1] issuer waiting for operands (full
// barriers)  [2] issuer waiting for an accumulator (epilogue not done)  [3] K stages issued  [4] leader's producer
// waiting for a free stage  [5] first epilogue warp of the leader waiting for a finished accumulator  [6] the same
// warp waiting for its staging buffers (output stores not yet read out of shared memory)  [7] tiles.
// Hand-over of the tensor pipe from one tile to the next, as sums of clock64 values over the tiles that have a
// successor (differences of the sums, divided by that number of tiles, are mean intervals): [9] the leader's first
// epilogue warp sees the tile finished  [10] it has the shared columns in registers and releases the accumulator
// [8] the issuer sees the release (the next tile's first MMA is issued right after); [13] / [12] / [11]: the epilogue
// warp past its tcgen05 fence / the loads of the first 64 columns issued / their data in registers.
// g_trace_no_loads != 0: after the first fill of the ring the producers only signal the stages instead of loading
// them (results are garbage): the stage time without any operand traffic into shared memory.
constexpr int kTraceClusters = 128;
constexpr int kTraceSlots = 16;
__device__ unsigned long long g_pair_trace[kTraceClusters][kTraceSlots];
__device__ int g_trace_no_loads;
__device__ __forceinline__ long long trace_clock() { return clock64(); }
#define NVFP_TRACE(...) __VA_ARGS__
#else
#define NVFP_TRACE(...)
#endif

// Tile number -> tile row and column.  Tiles are numbered down the rows of a BAND of p.band tile rows, column after
// column, band after band.  The host sizes a band so that its rows of A stay in L2 while all of B streams past them
// once (launch_pair): with whole columns of tiles and an A larger than L2, A would come from DRAM again for every
// two or three tile columns (M = N = 8192, K = 28672: 648 us in bands of 10 tile rows, 709-756 us in whole columns).
__device__ __forceinline__ void pair_tile_coords(const GemmParams& p, int tile, int& tm, int& tn) {
  const int per_band = p.band * p.tiles_n;
  const int b = tile / per_band, within = tile - b * per_band;
  const int rows = min(p.band, p.tiles_m - b * p.band);
  tn = within / rows;
  tm = b * p.band + (within - tn * rows);
}

template <bool MX, typename OutT, int OUT_MODE = kOutStoreAll>
__global__ void __launch_bounds__(kThreads, 1)
fp4_gemm_pair_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                     const __grid_constant__ CUtensorMap tmap_sfa, const __grid_constant__ CUtensorMap tmap_sfb,
                     const __grid_constant__ OutMaps out_maps, const int n_out, const int rows_per_owner,
                     const GemmParams p, const PeerSync sync, const GatherFp4 gq) {
  using C = PairCfg<MX>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C::kStages * C::kStageBytes + C::kStagingBytes + C::kSfStagingBytes);
  constexpr int kFull = 0, kEmpty = C::kStages, kAccFull = 2 * C::kStages, kAccEmpty = kAccFull + 1,
                kDrain = kAccEmpty + 1, kEpiStart = kDrain + 1, kEpiEnd = kEpiStart + 1, kNumBars = kEpiEnd + 1;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + kNumBars);
  volatile uint32_t* abort_flag = tmem_slot + 1;
  volatile uint32_t* never_set = tmem_slot + 2;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();          // 0 = leader
  const uint32_t smem_base = smem_u32(smem);
  auto bar = [&](int i) { return smem_u32(bars + i); };

  // number of this call among the calls that share the flag blocks (read by every thread before any epilogue warp of
  // this grid can finish, hence before the last one advances the stored count)
  uint32_t peer_seq = 0;
  if (sync.world > 1) {
    peer_seq = ld_acquire_sys(sync.flags[sync.rank] + 17) + 1u;
    if (blockIdx.x == 0 && threadIdx.x == 0)
      for (int r = 0; r < sync.world; ++r)
        if (r != sync.rank) st_release_sys(sync.flags[r] + sync.rank, peer_seq);     // ready[rank] on rank r
  }

  if (threadIdx.x == 0) {
    for (int i = 0; i < C::kStages; ++i) {
      mbar_init(bar(kFull + i), 1);     // armed by the leader's producer for the bytes of BOTH CTAs
      mbar_init(bar(kEmpty + i), 1);    // one commit from the leader's issuer
    }
    mbar_init(bar(kAccFull), 1);        // one commit from the leader's issuer
    mbar_init(bar(kAccEmpty), 8);       // 4 epilogue warps x 2 CTAs (used in the leader)
    mbar_init(bar(kDrain), 1);
    mbar_init(bar(kEpiStart), 4);       // the four epilogue warps of this CTA, once per tile (kOutFp4Gather)
    mbar_init(bar(kEpiEnd), 4);
    *abort_flag = 0;
    *never_set = 0;
    fence_mbar_init();
    prefetch_tensormap(&tmap_a);
    prefetch_tensormap(&tmap_b);
    prefetch_tensormap(&tmap_sfa);
    prefetch_tensormap(&tmap_sfb);
  }
  if (warp == 1) {
    tmem_alloc_pair(smem_u32(tmem_slot), kTmemCols);
    tmem_relinquish_alloc_permit_pair();
  }
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();                    // the peer's barriers and tensor memory exist from here on
  tc_fence_after_sync();
  if (p.release_next) griddep_launch_dependents();
  const uint32_t tmem_base = *tmem_slot;

  const int num_tiles = p.tiles_m * p.tiles_n;
  const int k_stages = (p.k + kStageK - 1) / kStageK;
  const int first_tile = (int)cluster_id_x();
  const int tile_step = (int)num_clusters_x();

  if (warp == 0) {
    // ------------------------------------------------------------ producer ---
    if (elect_one()) {
      uint32_t kc = 0;
      int ks0 = 0;
      bool ok = true;
      NVFP_TRACE(long long trace_producer_wait = 0;)
      if (p.after_producer && first_tile < num_tiles) {
        // Launched under the kernel that writes A, its scales and alpha: the ring's first fill fetches the B side
        // (which that kernel does not touch) at once and the A side after griddepcontrol.wait.
        int tm, tn;
        pair_tile_coords(p, first_tile, tm, tn);
        const int early = min(k_stages, C::kStages);
        for (int ks = 0; ks < early; ++ks) {
          const uint32_t st = smem_base + (uint32_t)ks * C::kStageBytes;
          const uint32_t full = map_to_cta(bar(kFull + ks), 0);
          if (rank == 0) mbar_arrive_expect_tx(bar(kFull + ks), 2 * C::kStageBytes);
          tma_load_2d_pair(st + C::kABytes, &tmap_b, full, ks * kStageKBytes, tn * kPairBN + (int)rank * 128);
          tma_load_3d_pair(st + C::kABytes + C::kBBytes + C::kSfaBytes, &tmap_sfb, full, 0,
                           ks * C::kChunksPerStage, tn * 2);
        }
        griddep_wait();
        for (int ks = 0; ks < early; ++ks) {
          const uint32_t st = smem_base + (uint32_t)ks * C::kStageBytes;
          const uint32_t full = map_to_cta(bar(kFull + ks), 0);
          tma_load_2d_pair(st, &tmap_a, full, ks * kStageKBytes, tm * kPairBM + (int)rank * 128);
          tma_load_3d_pair(st + C::kABytes + C::kBBytes, &tmap_sfa, full, 0, ks * C::kChunksPerStage,
                           tm * 2 + (int)rank);
        }
        kc = (uint32_t)early;
        ks0 = early;
      }
      for (int tile = first_tile; tile < num_tiles && ok; tile += tile_step, ks0 = 0) {
        int tm, tn;
        pair_tile_coords(p, tile, tm, tn);
        for (int ks = ks0; ks < k_stages; ++ks, ++kc) {
          const uint32_t s = kc % C::kStages, ph = (kc / C::kStages) & 1u;
          NVFP_TRACE(const long long tw0 = trace_clock();)
          if (!mbar_wait_bounded(bar(kEmpty + s), ph ^ 1u, abort_flag)) {
            *abort_flag = 1;
            atomicOr(p.status, kErrProducer);
            ok = false;
            break;
          }
          NVFP_TRACE(trace_producer_wait += trace_clock() - tw0;)
          const uint32_t st = smem_base + s * C::kStageBytes;
          const uint32_t full = map_to_cta(bar(kFull + s), 0);
          // Only the leader arms the barrier (CTA-local, no cluster-scope release on the hot path).  The
          // peer's bytes may arrive first: the transaction count goes negative for a moment, the phase
          // cannot complete before the leader's arrival.
          NVFP_TRACE(if (g_trace_no_loads && kc >= (uint32_t)C::kStages) {
            if (rank == 0) mbar_arrive(bar(kFull + s));
            continue;
          })
          if (rank == 0) mbar_arrive_expect_tx(bar(kFull + s), 2 * C::kStageBytes);
          tma_load_2d_pair(st, &tmap_a, full, ks * kStageKBytes, tm * kPairBM + (int)rank * 128);
          tma_load_2d_pair(st + C::kABytes, &tmap_b, full, ks * kStageKBytes, tn * kPairBN + (int)rank * 128);
          tma_load_3d_pair(st + C::kABytes + C::kBBytes, &tmap_sfa, full, 0, ks * C::kChunksPerStage,
                           tm * 2 + (int)rank);
          tma_load_3d_pair(st + C::kABytes + C::kBBytes + C::kSfaBytes, &tmap_sfb, full, 0,
                           ks * C::kChunksPerStage, tn * 2);
        }
      }
      NVFP_TRACE(if (rank == 0 && cluster_id_x() < kTraceClusters) g_pair_trace[cluster_id_x()][4] = (unsigned long long)trace_producer_wait;)
      if (!ok || *abort_flag) {
        // The loads already issued report to the leader's barriers, which this thread cannot wait
        // on from the peer CTA: give them a fixed, bounded time to land before the CTA may exit.
        const uint64_t t0 = global_timer_ns();
        while (global_timer_ns() - t0 < 200000ull) __nanosleep(1000);
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // -------------------------------------------------------------- issuer ---
    if (rank == 0 && elect_one()) {
      // This one thread feeds the tensor pipe of both SMs; whatever it does between two MMAs that the
      // pipe's small queue cannot cover shows up as idle tensor cycles.  Hence: stage index and phase
      // are carried instead of recomputed, descriptors are formed by adding constants, and the next
      // stage's barrier is polled once BEFORE the last MMAs of the current stage are queued.
      bool ok = true;
      int it = 0;
      uint32_t s = 0, ph = 0;
      bool next_ready = false;
      const uint32_t acc_full_0 = map_to_cta(bar(kAccFull), 0), acc_full_1 = map_to_cta(bar(kAccFull), 1);
      const uint32_t empty_0 = map_to_cta(bar(kEmpty), 0), empty_1 = map_to_cta(bar(kEmpty), 1);
      const uint64_t a_desc0 = make_smem_desc(smem_base, 16, 1024, 2);
      const uint64_t b_desc0 = make_smem_desc(smem_base + C::kABytes, 16, 1024, 2);
      const uint64_t sfa_desc0 = make_smem_desc(smem_base + C::kABytes + C::kBBytes, 0, 128, 0);
      const uint64_t sfb_desc0 = make_smem_desc(smem_base + C::kABytes + C::kBBytes + C::kSfaBytes, 0, 128, 0);
      const uint32_t sfa_tmem = tmem_base + C::kSfColBase, sfb_tmem = sfa_tmem + C::kSfaCols;
      const int tail_mmas = (p.k - (k_stages - 1) * kStageK + kMmaK - 1) / kMmaK;   // MMAs in the last stage
      NVFP_TRACE(long long trace_full = 0, trace_acc = 0, trace_stages = 0; const long long trace_t0 = trace_clock();
                 unsigned long long trace_handover = 0;)
      for (int tile = first_tile; tile < num_tiles && ok; tile += tile_step, ++it) {
        NVFP_TRACE(const long long ta0 = trace_clock();)
        if (!mbar_wait_bounded(bar(kAccEmpty), ((uint32_t)it & 1u) ^ 1u, abort_flag)) {
          *abort_flag = 1;
          atomicOr(p.status, kErrIssuer);
          break;
        }
        NVFP_TRACE(trace_acc += trace_clock() - ta0; if (it > 0) trace_handover += (unsigned long long)trace_clock();)
        const uint32_t d_tmem = tmem_base + ((it & 1) ? C::kOddAccCol : 0u);
        const bool more_tiles = tile + tile_step < num_tiles;
        for (int ks = 0; ks < k_stages; ++ks) {
          NVFP_TRACE(const long long tf0 = trace_clock();)
          if (!next_ready && !mbar_wait_bounded(bar(kFull + s), ph, abort_flag)) {
            *abort_flag = 1;
            atomicOr(p.status, kErrIssuer);
            ok = false;
            break;
          }
          NVFP_TRACE(if (!next_ready) trace_full += trace_clock() - tf0; ++trace_stages;)
          tc_fence_after_sync();
          const int mmas = ks == k_stages - 1 ? tail_mmas : kStageK / kMmaK;
          const uint64_t stage_off = (uint64_t)((s * C::kStageBytes) >> 4);
          const uint64_t a_desc = a_desc0 + stage_off, b_desc = b_desc0 + stage_off;
          const uint64_t sfa_desc = sfa_desc0 + stage_off, sfb_desc = sfb_desc0 + stage_off;
          const uint32_t s_next = s + 1 == (uint32_t)C::kStages ? 0u : s + 1;
          const uint32_t ph_next = s_next == 0 ? ph ^ 1u : ph;
          const bool has_next = more_tiles || ks + 1 < k_stages;
          next_ready = false;
          // One set of scale columns: tcgen05.cp and tcgen05.mma of one thread execute in issue order,
          // so a copy cannot overtake the earlier MMAs that read the columns it overwrites.
#pragma unroll
          for (int c = 0; c < C::kChunksPerStage; ++c) {
            if (c * C::kMmasPerChunk < mmas) {
              if (c == C::kChunksPerStage - 1 && has_next) next_ready = mbar_try_wait(bar(kFull + s_next), ph_next);
              tc_copy_sf_32x128b_warpx4_pair(sfa_tmem + 4 * c, sfa_desc + 32 * c);
              tc_copy_sf_32x128b_warpx4_pair(sfb_tmem + 8 * c, sfb_desc + 32 * c);
              tc_copy_sf_32x128b_warpx4_pair(sfb_tmem + 8 * c + 4, sfb_desc + 32 * (C::kChunksPerStage + c));
#pragma unroll
              for (int jj = 0; jj < C::kMmasPerChunk; ++jj) {
                const int j = c * C::kMmasPerChunk + jj;
                if (j < mmas) {
                  const uint32_t accumulate = (ks | j) != 0 ? 1u : 0u;
                  if (MX)
                    tc_mma_mxf4_pair(d_tmem, a_desc + 2 * j, b_desc + 2 * j,
                                     make_idesc_fp4_block_scaled(kPairBM, kPairBN, true, 2u * jj, 2u * jj),
                                     sfa_tmem + 4 * c, sfb_tmem + 8 * c, accumulate);
                  else
                    tc_mma_nvf4_pair(d_tmem, a_desc + 2 * j, b_desc + 2 * j,
                                     make_idesc_fp4_block_scaled(kPairBM, kPairBN, false),
                                     sfa_tmem + 4 * c, sfb_tmem + 8 * c, accumulate);
                }
              }
            }
          }
          // the stage is reusable in BOTH CTAs once these MMAs have read it
          tc_commit_pair(empty_0 + 8 * s);
          tc_commit_pair(empty_1 + 8 * s);
          s = s_next;
          ph = ph_next;
        }
        if (ok) {
          tc_commit_pair(acc_full_0);
          tc_commit_pair(acc_full_1);
        }
      }
      NVFP_TRACE(if (cluster_id_x() < kTraceClusters) {
        unsigned long long* t = g_pair_trace[cluster_id_x()];
        t[0] = (unsigned long long)(trace_clock() - trace_t0); t[1] = (unsigned long long)trace_full;
        t[2] = (unsigned long long)trace_acc; t[3] = (unsigned long long)trace_stages; t[7] = (unsigned long long)it;
        t[8] = trace_handover;
      })
      if (*abort_flag) {
        tc_commit_pair(map_to_cta(bar(kDrain), 0));
        mbar_wait_bounded(bar(kDrain), 0, never_set, 200000000ull);
      }
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------------ epilogue ---
    // Accumulator -> registers (tcgen05.ld) -> x alpha -> OutT -> swizzled staging buffer in shared
    // memory -> one TMA store per destination.  A warp owns 32 rows and stores 128 bytes of each per step.
    constexpr int kCols = 128 / (int)sizeof(OutT);          // columns per store: 64 (16-bit) or 32 (fp32)
    constexpr int kSteps = kPairBN / kCols;
    constexpr int kEarlySteps = 64 / kCols;                  // steps that cover the 48 shared columns
    const int q = warp & 3;
    if (p.after_producer) griddep_wait();   // alpha comes from the kernel before this one
    const float alpha = load_alpha(p);
    const OutT* bias = static_cast<const OutT*>(p.bias);
    uint32_t mx2_bits = 0;                       // running max |value stored| of this lane (pair of OutT)
    const bool track_amax = OUT_MODE == kOutStoreAll && sizeof(OutT) == 2 && p.amax_scratch != nullptr;
    const float out_gs = ((OUT_MODE == kOutFused || OUT_MODE == kOutFp4Gather) && p.out_gs) ? __ldg(p.out_gs) : 1.0f;
    const float rcp_out_gs = rcp_approx_ftz(out_gs), rcp6 = rcp_approx_ftz(6.0f);
    const uint32_t acc_empty_leader = map_to_cta(bar(kAccEmpty), 0);
    const uint32_t staging = smem_base + C::kStages * C::kStageBytes + (uint32_t)(warp - 2) * 2 * C::kStoreBufBytes;
    uint32_t store_count = 0;
    int it = 0;
    // destinations in other GPUs' memory are written only once their owners have announced ready (lane 0 decides:
    // it issues the stores)
    bool peers_asked = sync.world <= 1, remote_ok = true;
    NVFP_TRACE(long long trace_accfull = 0, trace_store = 0; unsigned long long trace_seen = 0, trace_released = 0, trace_ld_issued = 0, trace_loaded = 0, trace_fenced = 0, trace_first_ld = 0;)
    for (int tile = first_tile; tile < num_tiles; tile += tile_step, ++it) {
      int tm, tn;
      pair_tile_coords(p, tile, tm, tn);
      NVFP_TRACE(const long long te0 = trace_clock();)
      if (!__all_sync(0xffffffffu, mbar_wait_bounded(bar(kAccFull), (uint32_t)it & 1u, abort_flag))) {
        *abort_flag = 1;
        if (lane == 0) atomicOr(p.status, kErrEpilogue);
        break;
      }
      NVFP_TRACE(trace_accfull += trace_clock() - te0; if (tile + tile_step < num_tiles) trace_seen += (unsigned long long)trace_clock();)
      tc_fence_after_sync();
      NVFP_TRACE(if (tile + tile_step < num_tiles) trace_fenced += (unsigned long long)trace_clock();)
      const int row0 = tm * kPairBM + (int)rank * 128 + q * 32;
      const bool odd = (it & 1) != 0;
      const uint32_t t_row = tmem_base + (odd ? C::kOddAccCol : 0u) + ((uint32_t)(q * 32) << 16);
      bool bail = false;
#pragma unroll 1
      for (int i = 0; i < kSteps; ++i) {
        // Even tiles drain from the last columns down, odd tiles from the first up: either way the
        // columns shared with the other accumulator are read first, and the accumulator is handed
        // back as soon as they are in registers, so the next tile's MMAs start early.
        const int c = odd ? i : kSteps - 1 - i;
        uint32_t r[kCols];
#pragma unroll
        for (int h = 0; h < kCols / 32; ++h) {
          tmem_ld_32x32b_x32(t_row + c * kCols + h * 32, *reinterpret_cast<uint32_t(*)[32]>(&r[h * 32]));
          NVFP_TRACE(if (h == 0 && i == 0 && tile + tile_step < num_tiles) trace_first_ld += (unsigned long long)trace_clock();)
        }
        NVFP_TRACE(if (i == 0 && tile + tile_step < num_tiles) trace_ld_issued += (unsigned long long)trace_clock();)
        tmem_ld_wait();
        NVFP_TRACE(if (i == 0 && tile + tile_step < num_tiles) trace_loaded += (unsigned long long)trace_clock();)
        if (i == kEarlySteps - 1) {
          tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) mbar_arrive_remote(acc_empty_leader);
          NVFP_TRACE(if (tile + tile_step < num_tiles) trace_released += (unsigned long long)trace_clock();)
        }
        if constexpr (OUT_MODE == kOutFused) {
          if (p.act) finish_row_chunk<OutT, 64, true>(p, r, alpha, bias, row0 + lane, tn * kPairBN + c * kCols, out_gs, rcp_out_gs, rcp6);
          else finish_row_chunk<OutT, 64, false>(p, r, alpha, bias, row0 + lane, tn * kPairBN + c * kCols, out_gs, rcp_out_gs, rcp6);
          continue;
        }
        if constexpr (OUT_MODE == kOutFp4Gather) {
          // A warp's 32 rows x 256 columns of a tile are 32 x 128 bytes of packed nibbles: ONE 128-byte-swizzled box,
          // filled 32 bytes per row and step and stored once per destination when the tile is done (two boxes per
          // warp, alternating by tile).  The tile's scale bytes -- 128 rows x 16, four 512-byte chunks of the
          // swizzled layout, contiguous in memory -- are staged by the four warps together and leave as one bulk
          // copy per destination, issued by the first epilogue warp.
          static_assert(kCols == 64, "16-bit value type");
          const uint32_t fp4_buf = staging + (uint32_t)(it & 1) * C::kStoreBufBytes;
          const uint32_t sf_buf = smem_base + C::kStages * C::kStageBytes + C::kStagingBytes;
          if (i == 0) {
            // this warp's box of two tiles ago, and (first epilogue warp) the previous tile's scale copies, have
            // been read out of shared memory; all four warps know before anyone overwrites the scale chunks
            if (lane == 0) {
              bulk_wait_group_read<1>();
              mbar_arrive(bar(kEpiStart));
            }
            if (!__all_sync(0xffffffffu, mbar_wait_bounded(bar(kEpiStart), (uint32_t)it & 1u, abort_flag))) {
              *abort_flag = 1;
              if (lane == 0) atomicOr(p.status, kErrEpilogue);
              bail = true;
              break;
            }
          }
          uint2 qv[4];
          uint32_t sf_word;
          quantize_row_chunk_to_regs<OutT, 64>(p, r, alpha, bias, row0 + lane, tn * kPairBN + c * kCols, out_gs, rcp_out_gs,
                                               rcp6, qv, sf_word);
          st_shared_v4(fp4_buf + (uint32_t)lane * 128u + (uint32_t)(((2 * c) ^ (lane & 7)) << 4),
                       make_uint4(qv[0].x, qv[0].y, qv[1].x, qv[1].y));
          st_shared_v4(fp4_buf + (uint32_t)lane * 128u + (uint32_t)(((2 * c + 1) ^ (lane & 7)) << 4),
                       make_uint4(qv[2].x, qv[2].y, qv[3].x, qv[3].y));
          asm volatile("st.shared.b32 [%0], %1;" ::"r"(sf_buf + (uint32_t)c * 512u + (uint32_t)lane * 16u + (uint32_t)q * 4u),
                       "r"(sf_word) : "memory");
          if (i == kSteps - 1) {
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar(kEpiEnd));
            bool chunks_staged = true;
            if (warp == 2) chunks_staged = __all_sync(0xffffffffu, mbar_wait_bounded(bar(kEpiEnd), (uint32_t)it & 1u, abort_flag));
            if (lane == 0) {
              if (!peers_asked) {
                peers_asked = true;
                for (int rr = 0; rr < sync.world; ++rr)
                  if (rr != sync.rank && !wait_flag_reached(sync.flags[sync.rank] + rr, peer_seq, sync.limit_ns)) remote_ok = false;
                if (!remote_ok) atomicOr(p.status, kErrPeerWait);
              }
              const int n_store = remote_ok ? n_out : 1;
              if (warp == 2 && chunks_staged) {
                const int row_tile = tm * 2 + (int)rank, chunks = min(4, gq.k_tiles_slab - tn * 4);
                if (row_tile * 128 < p.m && chunks > 0) {
                  const int64_t off = ((int64_t)row_tile * gq.k_tiles_total + gq.k_tile0 + tn * 4) * 512;
                  for (int o = 0; o < n_store; ++o)
                    asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;"
                                 ::"l"(gq.sf[o] + off), "r"(sf_buf), "r"((uint32_t)chunks * 512u) : "memory");
                }
                bulk_commit_group();      // committed BEFORE this warp's box: the wait at the next tile's start covers it
              }
              for (int o = 0; o < n_store; ++o)
                tma_store_2d(&out_maps.map[o], fp4_buf, tn * (kPairBN / 2), row0);
              bulk_commit_group();
            }
            if (!chunks_staged) {
              *abort_flag = 1;
              if (lane == 0) atomicOr(p.status, kErrEpilogue);
              bail = true;
            }
          }
          continue;
        }
        // the buffer used two steps ago must have been read out by its TMA store
        const uint32_t buf = staging + (store_count & 1u) * C::kStoreBufBytes;
        NVFP_TRACE(const long long ts0 = trace_clock();)
        if (lane == 0) bulk_wait_group_read<1>();
        __syncwarp();
        NVFP_TRACE(trace_store += trace_clock() - ts0;)
#pragma unroll
        for (int j = 0; j < 8; ++j) {     // eight 16-byte pieces of this thread's 128-byte row
          constexpr int kPer = 16 / (int)sizeof(OutT);
          const int colj = tn * kPairBN + c * kCols + j * kPer;
          const uint4 o = scale_bias_pack<OutT>(&r[kPer * j], alpha, (bias && colj < p.n) ? bias + colj : nullptr);
          st_shared_v4(buf + (uint32_t)lane * 128u + (uint32_t)((j ^ (lane & 7)) << 4), o);
          if (track_amax && row0 + lane < p.m) absmax_fold<OutT>(mx2_bits, o);     // rows past m hold only the bias
        }
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) {
          if (!peers_asked) {
            peers_asked = true;
            for (int r = 0; r < sync.world; ++r)
              if (r != sync.rank && !wait_flag_reached(sync.flags[sync.rank] + r, peer_seq, sync.limit_ns)) remote_ok = false;
            if (!remote_ok) atomicOr(p.status, kErrPeerWait);
          }
          if constexpr (OUT_MODE == kOutScatterAdd) {
            const int owner = row0 / rows_per_owner;     // destinations are in rank order here
            if (owner < n_out && (remote_ok || sync.world <= 1 || owner == sync.rank))
              tma_reduce_add_2d(&out_maps.map[owner], buf, tn * kPairBN + c * kCols, row0 - owner * rows_per_owner);
          } else {
            // destination 0 is this GPU's own buffer, the others are the peers'
            const int n_store = remote_ok ? n_out : 1;
            for (int o = 0; o < n_store; ++o)
              tma_store_2d(&out_maps.map[o], buf, tn * kPairBN + c * kCols, row0);
          }
          bulk_commit_group();
        }
        ++store_count;
      }
      if (bail) break;
    }
    NVFP_TRACE(if (rank == 0 && warp == 2 && lane == 0 && cluster_id_x() < kTraceClusters) {
      g_pair_trace[cluster_id_x()][5] = (unsigned long long)trace_accfull;
      g_pair_trace[cluster_id_x()][6] = (unsigned long long)trace_store;
      g_pair_trace[cluster_id_x()][9] = trace_seen;
      g_pair_trace[cluster_id_x()][10] = trace_released;
      g_pair_trace[cluster_id_x()][11] = trace_loaded;
      g_pair_trace[cluster_id_x()][12] = trace_ld_issued;
      g_pair_trace[cluster_id_x()][13] = trace_fenced;
      g_pair_trace[cluster_id_x()][14] = trace_first_ld;
    })
    if (track_amax) absmax_finish<OutT>(p, mx2_bits, gridDim.x * 4u);
    if (lane == 0) bulk_wait_group<0>();    // all stores performed before the CTA may exit
    if (sync.world > 1 && lane == 0) {
      // this warp's stores have been performed; the last warp of the grid to get here tells the peers and waits for them
      __threadfence_system();
      uint32_t* mine = sync.flags[sync.rank];
      if (atomicAdd(mine + 16, 1u) == gridDim.x * 4u - 1u) {
        __threadfence_system();
        mine[16] = 0u;
        mine[17] = peer_seq;
        for (int r = 0; r < sync.world; ++r)
          if (r != sync.rank) st_release_sys(sync.flags[r] + 8 + sync.rank, peer_seq);   // done[rank] on rank r
        bool all = true;
        for (int r = 0; r < sync.world; ++r)
          if (r != sync.rank && !wait_flag_reached(mine + 8 + r, peer_seq, sync.limit_ns)) all = false;
        if (!all) atomicOr(p.status, kErrPeerWait);
      }
    }
    __syncwarp();
  }

  // -------------------------------------------------------------- common exit ---
  // Neither CTA may leave while the other can still signal its barriers or read its shared memory.
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();
  tc_fence_after_sync();
  if (warp == 1) tmem_dealloc_pair(tmem_base, kTmemCols);
}

// Scale tensor as a 3-D map: 512-byte chunk (128 x u32) | chunk index along K | 128-row tile.
inline int make_scale_map(CUtensorMap* map, const void* base, int64_t k_chunks, int64_t row_tiles,
                          int box_chunks, int box_tiles) {
  const cuuint64_t dims[3] = {128, (cuuint64_t)k_chunks, (cuuint64_t)row_tiles};
  const cuuint64_t strides[2] = {512, (cuuint64_t)k_chunks * 512};
  const cuuint32_t box[3] = {128, (cuuint32_t)box_chunks, (cuuint32_t)box_tiles};
  CUresult r = encode_tiled_cached(map, CU_TENSOR_MAP_DATA_TYPE_UINT32, 3, base, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_NONE,
                                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B);
  if (r != CUDA_SUCCESS) return fail(NVFP_ERR_CUDA, "cuTensorMapEncodeTiled (scales) failed with code %d", (int)r);
  return NVFP_OK;
}

// Row-major [rows, cols] output of OutT; box = 128 bytes x 32 rows, 128-byte swizzle.
template <typename OutT>
int make_output_map(CUtensorMap* map, void* base, int64_t rows, int64_t cols, int64_t ld) {
  const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)ld * sizeof(OutT)};
  const cuuint32_t box[2] = {(cuuint32_t)(128 / sizeof(OutT)), 32};
  const CUtensorMapDataType dt = sizeof(OutT) == 4 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                                 : std::is_same<OutT, __half>::value ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16
                                                                     : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  CUresult r = encode_tiled_cached(map, dt, 2, base, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE);
  if (r != CUDA_SUCCESS) return fail(NVFP_ERR_CUDA, "cuTensorMapEncodeTiled (output) failed with code %d", (int)r);
  return NVFP_OK;
}

// Row-major [rows, bytes_per_row] packed NVFP4 output (one rank's slab inside a wider matrix with row pitch ld_bytes);
// box = 128 bytes x 32 rows, 128-byte swizzle.
inline int make_packed_output_map(CUtensorMap* map, void* base, int64_t rows, int64_t bytes_per_row, int64_t ld_bytes) {
  const cuuint64_t dims[2] = {(cuuint64_t)bytes_per_row, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)ld_bytes};
  const cuuint32_t box[2] = {128, 32};
  CUresult r = encode_tiled_cached(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, base, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B,
                                   CU_TENSOR_MAP_L2_PROMOTION_NONE);
  if (r != CUDA_SUCCESS) return fail(NVFP_ERR_CUDA, "cuTensorMapEncodeTiled (packed output) failed with code %d", (int)r);
  return NVFP_OK;
}

// `outputs`: n_out destination matrices with leading dimension ld: [m, n] each (kOutStoreAll; outputs[0]
// is normally p.d) or [m / n_out, n] each (kOutScatterAdd).
template <bool MX, typename OutT, int OUT_MODE = kOutStoreAll>
int launch_pair(const GemmParams& base, const void* a, const void* b, void* const* outputs, int n_out,
                int64_t ld, int sm_count, cudaStream_t stream, const PeerSync* peer_sync = nullptr,
                const GatherFp4* gather_fp4 = nullptr) {
  using C = PairCfg<MX>;
  GemmParams p = base;
  p.tiles_m = (int)ceil_div(p.m, kPairBM);
  p.tiles_n = (int)ceil_div(p.n, kPairBN);
  {
    // With one band (A small enough to stay in L2) B is read from DRAM once; with A much larger than L2 and whole
    // columns of tiles, A would be read again for every two or three tile columns.
    const int64_t row_bytes = (int64_t)kPairBM * (p.k / 2 + p.k / 16);
    p.band = (int)std::max<int64_t>(1, std::min<int64_t>(p.tiles_m, kPairBandBytes / std::max<int64_t>(row_bytes, 1)));
  }
#ifdef NVFP_PAIR_TRACE
  if (const char* band = getenv("NVFP_TRACE_BAND")) p.band = std::max(1, std::min(p.tiles_m, atoi(band)));
#endif
  CUtensorMap map_a, map_b, map_sfa, map_sfb;
  if (int rc = make_operand_map(&map_a, a, p.m, p.k, 128)) return rc;
  if (int rc = make_operand_map(&map_b, b, p.n, p.k, 128)) return rc;
  if (int rc = make_scale_map(&map_sfa, p.sfa, p.sf_k_chunks, ceil_div(p.m, 128), C::kChunksPerStage, 1)) return rc;
  if (int rc = make_scale_map(&map_sfb, p.sfb, p.sf_k_chunks, ceil_div(p.n, 128), C::kChunksPerStage, 2)) return rc;
  OutMaps out_maps;
  memset(&out_maps, 0, sizeof(out_maps));
  const int rows_per_owner = OUT_MODE == kOutScatterAdd ? p.m / n_out : p.m;
  if constexpr (OUT_MODE == kOutFp4Gather) {
    // outputs[o]: where this rank's packed slab starts in destination o's [m, ld / 2]-byte matrix
    for (int o = 0; o < n_out; ++o)
      if (int rc = make_packed_output_map(&out_maps.map[o], outputs[o], p.m, p.n / 2, ld / 2)) return rc;
  } else if constexpr (OUT_MODE != kOutFused) {
    for (int o = 0; o < n_out; ++o)
      if (int rc = make_output_map<OutT>(&out_maps.map[o], outputs[o], rows_per_owner, p.n, ld)) return rc;
  }
  auto kernel = fp4_gemm_pair_kernel<MX, OutT, OUT_MODE>;
  if (int rc = ensure_dynamic_smem(kernel, (int)C::kSmemBytes)) return rc;
  const int64_t tiles = (int64_t)p.tiles_m * p.tiles_n;
  unsigned pairs = (unsigned)std::min<int64_t>(tiles, sm_count / 2);
#ifdef NVFP_PAIR_TRACE
  // instrumented build only: fewer CTA pairs, to see how a pair's stage time depends on how many pairs pull operands
  if (const char* cap = getenv("NVFP_TRACE_MAX_PAIRS")) pairs = std::max(1u, std::min(pairs, (unsigned)atoi(cap)));
  {
    const char* no_loads = getenv("NVFP_TRACE_NO_LOADS");
    const int flag = no_loads && atoi(no_loads) != 0;
    NVFP_CUDA(cudaMemcpyToSymbolAsync(g_trace_no_loads, &flag, sizeof(flag), 0, cudaMemcpyHostToDevice, stream));
  }
#endif
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * pairs);
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = C::kSmemBytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = p.after_producer ? 2 : 1;
  PeerSync sync;
  memset(&sync, 0, sizeof(sync));
  if (peer_sync) sync = *peer_sync;
  GatherFp4 gq;
  memset(&gq, 0, sizeof(gq));
  if (gather_fp4) gq = *gather_fp4;
  NVFP_CUDA(cudaLaunchKernelEx(&cfg, kernel, map_a, map_b, map_sfa, map_sfb, out_maps, n_out, rows_per_owner, p, sync, gq));
  return NVFP_OK;
}
