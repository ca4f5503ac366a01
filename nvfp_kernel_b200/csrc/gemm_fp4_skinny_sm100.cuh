// Block-scaled FP4 GEMM for few activation rows (decode, M <= 128).  Included by
// gemm_fp4_sm100.cu inside namespace nvfp::<anonymous>.
//
// With a handful of tokens the product is bound by streaming the weights once, and the
// reference's answer -- the same 128-row tile kernel, no split-K
// (kernel/nvfp4_scaled_mm_sm120_kernels.cu:190-220) -- leaves most SMs idle.  Here:
//   * operands are swapped: the 128 rows of the MMA are WEIGHT rows, the MMA's N is the token count
//     (rounded up to 16), so a stage holds 16 KB of weights and only NT x 128 bytes of activations;
//   * K is split over a cluster of up to 4 CTAs; each computes a partial [128 weight rows x NT tokens]
//     in tensor memory, the non-leaders write theirs into the leader's shared memory (distributed
//     shared memory, plain st.shared::cluster), the leader adds, scales by alpha and stores.  No
//     global scratch, no second kernel, no atomics.
#pragma once

// Measured on B200 inside a CUDA graph (warm L2), M=16: N=4096,K=14336 takes 14.4 us here against 25 us with
// the tile kernel; at K=4096 (N=4096: 9.6 vs 9.2 us, N=28672: 21.7 vs 20.6 us) there is nothing to gain, so the
// dispatcher only comes here for long K and few weight tiles.
constexpr int kSkinnyMaxTokens = 64;
constexpr uint32_t kSkinnyReduceBytes = 64 * 1024;   // leader's buffer for the peers' partial sums
constexpr uint32_t kSkinnyTmemCols = 256;

template <bool MX>
struct SkinnyCfg {
  static constexpr int kChunksPerStage = MX ? 2 : 4;
  static constexpr int kMmasPerChunk = MX ? 2 : 1;
  static constexpr uint32_t kWBytes = 128 * kStageKBytes;            // weight tile of a stage
  static constexpr uint32_t kXBytesMax = kSkinnyMaxTokens * kStageKBytes;
  static constexpr uint32_t kSfBytes = kChunksPerStage * 512;        // per operand
  static constexpr uint32_t kSfColBase = 128;                        // accumulator: columns [0, NT)
};

struct SkinnyParams {
  GemmParams g;
  int nt;               // MMA N = tokens rounded up to 16
  int split;            // cluster size = K splits
  int stages_per_rank;  // K stages (of 256 elements) each rank of a cluster processes
  int num_stages;       // pipeline depth
  uint32_t stage_bytes;
};

__device__ __forceinline__ void st_cluster_f32(uint32_t cluster_addr, float v) {
  asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(cluster_addr), "f"(v) : "memory");
}

template <bool MX, typename OutT>
__global__ void __launch_bounds__(kThreads)
fp4_gemm_skinny_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_x,
                       const SkinnyParams sp) {
  using C = SkinnyCfg<MX>;
  const GemmParams& p = sp.g;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  // [reduce buffer 64 KB][stages][barriers]
  float* reduce_buf = reinterpret_cast<float*>(smem);
  uint8_t* stage0 = smem + kSkinnyReduceBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(stage0 + sp.num_stages * sp.stage_bytes);
  const int kFull = 0, kEmpty = sp.num_stages, kAccFull = 2 * sp.num_stages, kNumBars = kAccFull + 1;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + kNumBars);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const int n_tile = (int)cluster_id_x();
  const uint32_t stage_base = smem_u32(stage0);
  auto bar = [&](int i) { return smem_u32(bars + i); };
  const uint32_t x_bytes = (uint32_t)sp.nt * kStageKBytes;
  const uint32_t off_x = C::kWBytes, off_sfw = C::kWBytes + x_bytes, off_sfx = off_sfw + C::kSfBytes;

  if (threadIdx.x == 0) {
    for (int i = 0; i < sp.num_stages; ++i) {
      mbar_init(bar(kFull + i), 1);
      mbar_init(bar(kEmpty + i), 1);
    }
    mbar_init(bar(kAccFull), 1);
    *abort_flag = 0;
    fence_mbar_init();
    prefetch_tensormap(&tmap_w);
    prefetch_tensormap(&tmap_x);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), kSkinnyTmemCols);
    tmem_relinquish_alloc_permit();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  const int total_stages = (p.k + kStageK - 1) / kStageK;
  const int ks_begin = min((int)rank * sp.stages_per_rank, total_stages);
  const int ks_end = min(ks_begin + sp.stages_per_rank, total_stages);
  const int my_stages = ks_end - ks_begin;

  if (warp == 0) {
    // ------------------------------------------------------------ producer ---
    if (elect_one()) {
      for (int i = 0; i < my_stages; ++i) {
        const int ks = ks_begin + i;
        const uint32_t s = (uint32_t)i % sp.num_stages, ph = ((uint32_t)i / sp.num_stages) & 1u;
        if (!mbar_wait_bounded(bar(kEmpty + s), ph ^ 1u, abort_flag)) {
          *abort_flag = 1;
          atomicOr(p.status, kErrProducer);
          break;
        }
        const int chunks = min(C::kChunksPerStage, p.sf_k_chunks - ks * C::kChunksPerStage);
        const uint32_t sf_bytes = (uint32_t)chunks * 512u;
        const uint32_t st = stage_base + s * sp.stage_bytes;
        mbar_arrive_expect_tx(bar(kFull + s), C::kWBytes + x_bytes + 2 * sf_bytes);
        tma_load_2d(st, &tmap_w, bar(kFull + s), ks * kStageKBytes, n_tile * 128);
        tma_load_2d(st + off_x, &tmap_x, bar(kFull + s), ks * kStageKBytes, 0);
        const int64_t chunk0 = (int64_t)ks * C::kChunksPerStage;
        bulk_load(st + off_sfw, p.sfb + ((int64_t)n_tile * p.sf_k_chunks + chunk0) * 512, sf_bytes, bar(kFull + s));
        bulk_load(st + off_sfx, p.sfa + chunk0 * 512, sf_bytes, bar(kFull + s));
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // -------------------------------------------------------------- issuer ---
    if (elect_one()) {
      const uint32_t sfw_tmem = tmem_base + C::kSfColBase, sfx_tmem = sfw_tmem + 16;
      bool ok = true;
      for (int i = 0; i < my_stages && ok; ++i) {
        const int ks = ks_begin + i;
        const uint32_t s = (uint32_t)i % sp.num_stages, ph = ((uint32_t)i / sp.num_stages) & 1u;
        if (!mbar_wait_bounded(bar(kFull + s), ph, abort_flag)) {
          *abort_flag = 1;
          atomicOr(p.status, kErrIssuer);
          ok = false;
          break;
        }
        tc_fence_after_sync();
        const int chunks = min(C::kChunksPerStage, p.sf_k_chunks - ks * C::kChunksPerStage);
        const int mmas = min(kStageK / kMmaK, (p.k - ks * kStageK + kMmaK - 1) / kMmaK);
        const uint32_t st = stage_base + s * sp.stage_bytes;
        const uint64_t w_desc = make_smem_desc(st, 16, 1024, 2);
        const uint64_t x_desc = make_smem_desc(st + off_x, 16, 1024, 2);
        // tiny MMAs are latency-bound: queue all scale copies of the stage first (into one of two
        // alternating sets of columns), then the MMAs back to back
        const uint32_t slot = (uint32_t)(i & 1) * 32u;
        for (int c = 0; c < chunks; ++c) {
          tc_copy_sf_32x128b_warpx4(sfw_tmem + slot + 4 * c, make_smem_desc(st + off_sfw + c * 512, 0, 128, 0));
          tc_copy_sf_32x128b_warpx4(sfx_tmem + slot + 4 * c, make_smem_desc(st + off_sfx + c * 512, 0, 128, 0));
        }
        for (int j = 0; j < mmas; ++j) {
          const int c = j / C::kMmasPerChunk, jj = j % C::kMmasPerChunk;
          const uint32_t accumulate = (i | j) != 0 ? 1u : 0u;
          const uint64_t koff = (uint64_t)((j * (kMmaK / 2)) >> 4);
          if (MX)
            tc_mma_mxf4(tmem_base, w_desc + koff, x_desc + koff,
                        make_idesc_fp4_block_scaled(128, sp.nt, true, 2u * jj, 2u * jj), sfw_tmem + slot + 4 * c,
                        sfx_tmem + slot + 4 * c, accumulate);
          else
            tc_mma_nvf4(tmem_base, w_desc + koff, x_desc + koff, make_idesc_fp4_block_scaled(128, sp.nt, false),
                        sfw_tmem + slot + 4 * c, sfx_tmem + slot + 4 * c, accumulate);
        }
        tc_commit(bar(kEmpty + s));
      }
      if (ok) tc_commit(bar(kAccFull));
    }
    __syncwarp();
  }

  // ------------------------------------------------- partial sums -> leader ---
  // Epilogue warps of every rank pull their partial out of tensor memory; non-leaders push it
  // into the leader's reduce buffer laid out [rank-1][token][weight row].
  const bool epi = warp >= 2;
  const int q = warp & 3;
  const int wrow = q * 32 + lane;                 // weight row within the tile = accumulator lane
  bool have_acc = false;
  if (epi && my_stages > 0) {
    have_acc = __all_sync(0xffffffffu, mbar_wait_bounded(bar(kAccFull), 0, abort_flag));
    if (!have_acc) {
      *abort_flag = 1;
      if (lane == 0) atomicOr(p.status, kErrEpilogue);
    }
    tc_fence_after_sync();
  }
  const uint32_t t_row = tmem_base + ((uint32_t)(q * 32) << 16);
  if (epi && rank != 0) {
    const uint32_t dst0 = map_to_cta(smem_u32(reduce_buf), 0) + ((rank - 1) * (uint32_t)sp.nt * 128u + (uint32_t)wrow) * 4u;
    for (int c = 0; c < sp.nt; c += 16) {
      uint32_t r[16];
      if (have_acc) {
        asm volatile(
            "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
            : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
              "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
            : "r"(t_row + c)
            : "memory");
        tmem_ld_wait();
      } else {
#pragma unroll
        for (int t = 0; t < 16; ++t) r[t] = 0u;
      }
#pragma unroll
      for (int t = 0; t < 16; ++t) st_cluster_f32(dst0 + (uint32_t)(c + t) * 512u, __uint_as_float(r[t]));
    }
  }
  // all partials are in the leader's shared memory after this barrier (release / acquire at cluster scope)
  tc_fence_before_sync();
  cluster_sync_all();
  tc_fence_after_sync();
  if (epi && rank == 0) {
    const float alpha = p.alpha ? __ldg(p.alpha) : 1.0f;
    OutT* d = static_cast<OutT*>(p.d);
    const int n_global = n_tile * 128 + wrow;
    for (int c = 0; c < sp.nt; c += 16) {
      uint32_t r[16];
      if (have_acc) {
        asm volatile(
            "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
            : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
              "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
            : "r"(t_row + c)
            : "memory");
        tmem_ld_wait();
      } else {
#pragma unroll
        for (int t = 0; t < 16; ++t) r[t] = 0u;
      }
#pragma unroll
      for (int t = 0; t < 16; ++t) {
        float acc = __uint_as_float(r[t]);
        for (int pr = 0; pr < sp.split - 1; ++pr) acc += reduce_buf[(pr * sp.nt + c + t) * 128 + wrow];
        const int tok = c + t;
        if (tok < p.m && n_global < p.n) {
          const float v = acc * alpha;
          if constexpr (sizeof(OutT) == 4) d[(int64_t)tok * p.n + n_global] = v;
          else if constexpr (std::is_same<OutT, __half>::value) d[(int64_t)tok * p.n + n_global] = __float2half_rn(v);
          else d[(int64_t)tok * p.n + n_global] = __float2bfloat16_rn(v);
        }
      }
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  if (warp == 1) tmem_dealloc(tmem_base, kSkinnyTmemCols);
}

template <bool MX, typename OutT>
int launch_skinny(const GemmParams& base, const void* a, const void* b, int sm_count, cudaStream_t stream) {
  using C = SkinnyCfg<MX>;
  SkinnyParams sp{};
  sp.g = base;
  const int m = base.m, n = base.n, k = base.k;
  sp.nt = (int)round_up(m, 16);
  const int n_tiles = (int)ceil_div(n, 128);
  const int total_stages = (int)ceil_div(k, kStageK);
  // K split: enough CTAs to cover the SMs, at least two stages per rank, and the peers' partial sums
  // must fit the leader's reduce buffer
  int split = 1;
  while (split < 4 && n_tiles * split < sm_count && total_stages / (split * 2) >= 2 &&
         (uint32_t)sp.nt * (uint32_t)(split * 2 - 1) * 512u <= kSkinnyReduceBytes)
    split *= 2;
  sp.split = split;
  sp.stages_per_rank = (int)ceil_div(total_stages, split);
  sp.stage_bytes = (uint32_t)round_up(C::kWBytes + (uint32_t)sp.nt * kStageKBytes + 2 * C::kSfBytes, 1024);
  sp.num_stages = (int)std::min<int64_t>(sp.stages_per_rank, (kSmemLimit - 2048 - kSkinnyReduceBytes) / sp.stage_bytes);
  sp.num_stages = std::max(1, std::min(sp.num_stages, 8));
  const uint32_t smem_bytes = kSkinnyReduceBytes + (uint32_t)sp.num_stages * sp.stage_bytes + 2048;
  CUtensorMap map_w, map_x;
  if (int rc = make_operand_map(&map_w, b, n, k, 128)) return rc;
  if (int rc = make_operand_map(&map_x, a, m, k, sp.nt)) return rc;
  auto kernel = fp4_gemm_skinny_kernel<MX, OutT>;
  NVFP_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_bytes));
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)(n_tiles * split));
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = smem_bytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = (unsigned)split;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  NVFP_CUDA(cudaLaunchKernelEx(&cfg, kernel, map_w, map_x, sp));
  return NVFP_OK;
}
