// Block-scaled FP4 GEMM for few activation rows (decode, M <= 128).  Included by
// gemm_fp4_sm100.cu inside namespace nvfp::<anonymous>.
//
// With a handful of tokens the product is bound by streaming the weights once, and the
// reference's answer -- the same 128-row tile kernel, no split-K
// (kernel/nvfp4_scaled_mm_sm120_kernels.cu:190-220) -- leaves most SMs idle.  Here:
//   * operands are swapped: the 128 rows of the MMA are WEIGHT rows, the MMA's N is the token count
//     (rounded up to 16), so shared memory holds weights, not padding;
//   * a pipeline stage covers 1024 elements of K (512 above 64 tokens): four (two) 128-byte-swizzled boxes per
//     operand, so every weight row contributes 512 (256) contiguous bytes per stage, and the issuer pays one
//     barrier round trip per 16 (8) MMAs; all scale copies of a stage are queued before its MMAs (a barrier
//     per box measured 60 % slower per stage);
//   * with more weight tiles than SMs (and at most 32 tokens) the kernel is persistent: every CTA takes the same
//     number of tiles, its ring runs on across tile boundaries and the MMAs alternate between two accumulators, so
//     one tile's epilogue and the next tile's first loads overlap (N = 57344, K = 8192, 16 tokens: 50 us against
//     69 us as three and a bit waves of one-tile CTAs).  L2 prefetches of the weights ahead of the ring, by the
//     idle epilogue warps or rolling in the producer warp, measured neutral on one-tile shapes and 10 % slower here,
//     and a prefetch through the TMA unit halved the load rate: there are none;
//   * K is split over a cluster of CTAs; each computes a partial [128 weight rows x NT tokens] in tensor
//     memory.  The tokens are divided among "owners" -- the leader alone, or every rank when each can get a
//     multiple of 16 tokens -- and every rank sends each owner that owner's tokens of its partial: staged in its
//     own (drained) shared memory, then one bulk copy per warp and owner, shared memory to shared memory inside
//     the cluster, completion on an mbarrier of the owner.  An owner adds what it receives to its own partial,
//     scales by alpha, adds the bias and stores its tokens.  No global scratch, no second kernel, no atomics.
//   * the owner's epilogue can also apply the gated activation (a warp's 32 weight rows are 16 gate rows and their
//     16 up rows: lane l reads its up value from lane l + 16) and quantize the result to NVFP4 from the staging
//     tile, as the other two kernels do from registers.
#pragma once

constexpr int kSkinnyMaxTokens = 128;
constexpr int kSkinnyMaxSplit = 8;
constexpr uint32_t kSkinnyTmemCols = 256;
constexpr uint32_t kSkinnyOutTileBytes = 16 * 128 * 4;            // output staging: 16 tokens x 128 columns fp32
constexpr uint32_t kSkinnyAccCols = 128;                          // accumulator: columns [0, NT)

// BOXES: 256-element K boxes per stage.
template <bool MX, int BOXES>
struct SkinnyCfg {
  static constexpr int kStageElems = BOXES * kStageK;             // elements of K per stage
  static constexpr int kChunksPerBox = MX ? 2 : 4;                // 512-byte scale chunks per 256 elements of K
  static constexpr int kChunksPerStage = BOXES * kChunksPerBox;
  static constexpr int kMmasPerChunk = MX ? 2 : 1;
  static constexpr uint32_t kWBoxBytes = 128 * kStageKBytes;      // 16 KB
  static constexpr uint32_t kSfBytes = kChunksPerStage * 512;     // per operand per stage
  static constexpr uint32_t kSfwCol = kSkinnyAccCols;             // weight scales: 4 columns per chunk
  static constexpr uint32_t kSfxCol = kSfwCol + 4 * kChunksPerStage;
  static_assert(kSfxCol + 4 * kChunksPerStage <= kSkinnyTmemCols, "tensor memory budget");
};

struct SkinnyParams {
  GemmParams g;
  int nt;               // MMA N = tokens rounded up (to 16, or to 16 x owners)
  int split;            // cluster size = K splits
  int owners;           // ranks that reduce and store: 1 (the leader) or split (rank r owns tokens [r * tok, (r + 1) * tok))
  int tok;              // tokens per owner = nt / owners, a multiple of 16
  int stages_per_rank;  // stages each rank of a cluster processes
  int num_stages;       // pipeline depth
  uint32_t stage_bytes;
  int after_producer;      // launched with programmatic stream serialization behind the kernel that writes the
                           // activation operand, its scales and alpha: weights may be fetched before that kernel
                           // has finished, everything it writes only after griddepcontrol.wait
  // Byte offsets from the start of shared memory.  After the main loop the stage area [0, ring) is dead and holds,
  // from 0, the partial sums this rank stages for sending; behind them the output staging tile; the buffer this
  // rank receives into lies behind the ring when there is room (recv_behind_ring), else behind those two.
  uint32_t out_tile_offset;
  uint32_t recv_offset;
  int recv_behind_ring;
  uint32_t bars_offset;    // barriers, behind everything else
  // More weight tiles than SMs (then split == 1): a CTA works through tiles blockIdx.x, blockIdx.x + gridDim.x, ...
  // with the ring running on across tile boundaries and two accumulators, so that one tile's epilogue and the next
  // tile's first loads cost no time of their own.  The staging tile then lies behind the ring, which is never drained.
  int persistent;
};

// Partial sums travel as [128 weight rows][tok + 4] fp32 per (sender, owner) pair.  The 4 floats of padding make the
// row stride an odd number of 16-byte units, so 32 lanes reading one float4 each from consecutive rows hit distinct banks.
__host__ __device__ constexpr uint32_t skinny_block_ld(int tok) { return (uint32_t)tok + 4u; }
__host__ __device__ constexpr uint32_t skinny_block_bytes(int tok) { return 128u * skinny_block_ld(tok) * 4u; }

__device__ __forceinline__ void tmem_ld_32x32b_x16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}

template <bool MX, typename OutT, int BOXES>
__global__ void __launch_bounds__(kThreads)
fp4_gemm_skinny_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_x,
                       const SkinnyParams sp) {
  using C = SkinnyCfg<MX, BOXES>;
  const GemmParams& p = sp.g;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  // [stages ...][receive buffer, when it is behind the ring | staging tile, when persistent][barriers]
  const uint32_t block_bytes = skinny_block_bytes(sp.tok);                  // one sender's tokens for one owner
  const uint32_t recv_bytes = (uint32_t)(sp.split - 1) * block_bytes;
  const uint32_t ld = skinny_block_ld(sp.tok);
  float* recv_buf = reinterpret_cast<float*>(smem + sp.recv_offset);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + sp.bars_offset);
  const int kFull = 0, kEmpty = sp.num_stages, kAccFull = 2 * sp.num_stages, kAccEmpty = kAccFull + 2, kReduce = kAccEmpty + 2;
  const int kNumBars = kReduce + 1;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + kNumBars);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = sp.split > 1 ? cluster_ctarank() : 0u;
  const int tile0 = sp.split > 1 ? (int)cluster_id_x() : (int)blockIdx.x;
  const int tile_stride = sp.persistent ? (int)gridDim.x : 0;
  const int my_tiles = sp.persistent ? (p.sfb_row_tiles - tile0 + tile_stride - 1) / tile_stride : 1;
  const bool owner = (int)rank < sp.owners;
  const uint32_t stage_base = smem_u32(smem);
  auto bar = [&](int i) { return smem_u32(bars + i); };
  const uint32_t x_box_bytes = (uint32_t)sp.nt * kStageKBytes;
  const uint32_t off_x = BOXES * C::kWBoxBytes;
  const uint32_t off_sfw = off_x + BOXES * x_box_bytes, off_sfx = off_sfw + C::kSfBytes;

  const int total_stages = (p.k + C::kStageElems - 1) / C::kStageElems;
  const int ks_begin = min((int)rank * sp.stages_per_rank, total_stages);
  const int ks_end = min(ks_begin + sp.stages_per_rank, total_stages);
  const int my_stages = ks_end - ks_begin;
  const int k_boxes_total = (p.k + kStageK - 1) / kStageK;
  // Stages are counted through all of this CTA's tiles: stage g belongs to tile g / my_stages.
  const int total_g = my_tiles * my_stages;
  constexpr uint32_t kAccBufCols = 64;            // second accumulator (persistent: at most 32 tokens)

  // Loads of stage g into ring slot g % num_stages, all reported to the slot's one barrier.  `what` selects
  // the weight side (which also arms the barrier with the bytes of both sides), the activation side, or both.
  constexpr int kWeights = 1, kActivations = 2;
  auto load_stage = [&](int g, int what) {
    const int n_tile = tile0 + (g / my_stages) * tile_stride;
    const uint8_t* sfw_tile = p.sfb + (int64_t)n_tile * p.sf_k_chunks * 512;
    const int ks = ks_begin + g % my_stages;
    const uint32_t s = (uint32_t)g % sp.num_stages;
    const uint32_t st = stage_base + s * sp.stage_bytes;
    const int boxes = min(BOXES, k_boxes_total - ks * BOXES);
    const int chunk0 = ks * C::kChunksPerStage;
    const uint32_t sf_bytes = (uint32_t)min(C::kChunksPerStage, p.sf_k_chunks - chunk0) * 512u;
    const uint32_t full = bar(kFull + (int)s);
    if (what & kWeights) {
      mbar_arrive_expect_tx(full, (uint32_t)boxes * (C::kWBoxBytes + x_box_bytes) + 2 * sf_bytes);
      for (int b = 0; b < boxes; ++b)
        tma_load_2d(st + b * C::kWBoxBytes, &tmap_w, full, (ks * BOXES + b) * kStageKBytes, n_tile * 128);
      bulk_load(st + off_sfw, sfw_tile + (int64_t)chunk0 * 512, sf_bytes, full);
    }
    if (what & kActivations) {
      for (int b = 0; b < boxes; ++b)
        tma_load_2d(st + off_x + b * x_box_bytes, &tmap_x, full, (ks * BOXES + b) * kStageKBytes, 0);
      bulk_load(st + off_sfx, p.sfa + (int64_t)chunk0 * 512, sf_bytes, full);
    }
  };
  if (warp == 0) {
    // The producer thread initialises the barriers itself and starts the first loads before the rest of
    // the CTA (tensor memory allocation, the other warps) is ready.
    if (elect_one()) {
      for (int i = 0; i < kAccFull; ++i) mbar_init(bar(i), 1);
      for (int i = 0; i < 2; ++i) {
        mbar_init(bar(kAccFull + i), 1);
        mbar_init(bar(kAccEmpty + i), 4);          // one arrival per epilogue warp
      }
      mbar_init(bar(kReduce), 1);
      *abort_flag = 0;
      fence_mbar_init();
      fence_proxy_async_smem();
      if (sp.split > 1 && owner) mbar_arrive_expect_tx(bar(kReduce), recv_bytes);
      prefetch_tensormap(&tmap_w);
      prefetch_tensormap(&tmap_x);
      const int first = min(total_g, sp.num_stages);
      if (sp.after_producer) {
        // the weights do not depend on the kernel before this one: fetch them while it still runs
        for (int i = 0; i < first; ++i) load_stage(i, kWeights);
        griddep_wait();
        for (int i = 0; i < first; ++i) load_stage(i, kActivations);
      } else {
        for (int i = 0; i < first; ++i) load_stage(i, kWeights | kActivations);
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), kSkinnyTmemCols);
    tmem_relinquish_alloc_permit();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  if (p.release_next) griddep_launch_dependents();
  // With receive buffers behind the rings every rank is ready for the others' partial sums from here on.
  if (sp.split > 1 && sp.recv_behind_ring) cluster_arrive();

  if (warp == 0) {
    // ------------------------------------------------------------ producer ---
    if (elect_one()) {
      for (int g = sp.num_stages; g < total_g; ++g) {
        const uint32_t s = (uint32_t)g % sp.num_stages, ph = ((uint32_t)g / sp.num_stages) & 1u;
        if (!mbar_wait_bounded(bar(kEmpty + s), ph ^ 1u, abort_flag)) {
          *abort_flag = 1;
          atomicOr(p.status, kErrProducer);
          break;
        }
        load_stage(g, kWeights | kActivations);
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // -------------------------------------------------------------- issuer ---
    if (elect_one()) {
      const uint32_t sfw_tmem = tmem_base + C::kSfwCol, sfx_tmem = tmem_base + C::kSfxCol;
      const uint32_t idesc0 = make_idesc_fp4_block_scaled(128, sp.nt, MX, 0u, 0u);
      const uint32_t idesc1 = MX ? make_idesc_fp4_block_scaled(128, sp.nt, true, 2u, 2u) : idesc0;
      for (int g = 0; g < total_g; ++g) {
        const int j = g / my_stages, i = g % my_stages;
        const int ks = ks_begin + i;
        const uint32_t s = (uint32_t)g % sp.num_stages, ph = ((uint32_t)g / sp.num_stages) & 1u;
        const uint32_t st = stage_base + s * sp.stage_bytes;
        const int boxes = min(BOXES, k_boxes_total - ks * BOXES);
        const uint32_t acc = tmem_base + (uint32_t)(j & 1) * kAccBufCols;
        if (i == 0 && j >= 2) {
          // the epilogue has read this accumulator's previous tile
          if (!mbar_wait_bounded(bar(kAccEmpty + (j & 1)), (uint32_t)((j >> 1) - 1) & 1u, abort_flag)) {
            *abort_flag = 1;
            atomicOr(p.status, kErrIssuer);
            break;
          }
          tc_fence_after_sync();
        }
        if (!mbar_wait_bounded(bar(kFull + (int)s), ph, abort_flag)) {
          *abort_flag = 1;
          atomicOr(p.status, kErrIssuer);
          break;
        }
        tc_fence_after_sync();
        const int chunk0 = ks * C::kChunksPerStage;
        const int chunks = min(C::kChunksPerStage, p.sf_k_chunks - chunk0);
        // one set of scale columns per position in the stage: the tensor pipe runs one thread's copies and
        // MMAs in issue order, so a later stage's copies cannot overtake this stage's MMAs
        const uint64_t sfw_desc = make_smem_desc(st + off_sfw, 0, 128, 0);
        const uint64_t sfx_desc = make_smem_desc(st + off_sfx, 0, 128, 0);
        for (int c = 0; c < chunks; ++c) {
          tc_copy_sf_32x128b_warpx4(sfw_tmem + 4 * c, sfw_desc + (uint64_t)(c * 32));
          tc_copy_sf_32x128b_warpx4(sfx_tmem + 4 * c, sfx_desc + (uint64_t)(c * 32));
        }
        for (int b = 0; b < boxes; ++b) {
          const int mmas = min(kStageK / kMmaK, (p.k - (ks * BOXES + b) * kStageK + kMmaK - 1) / kMmaK);
          const uint64_t w_desc = make_smem_desc(st + b * C::kWBoxBytes, 16, 1024, 2);
          const uint64_t x_desc = make_smem_desc(st + off_x + b * x_box_bytes, 16, 1024, 2);
          const uint32_t bcol = 4u * (uint32_t)(b * C::kChunksPerBox);
          for (int j = 0; j < mmas; ++j) {
            const int c = j / C::kMmasPerChunk;
            const uint32_t accumulate = (i | b | j) != 0 ? 1u : 0u;
            if (MX)
              tc_mma_mxf4(acc, w_desc + (uint64_t)(2 * j), x_desc + (uint64_t)(2 * j), (j & 1) ? idesc1 : idesc0,
                          sfw_tmem + bcol + 4 * c, sfx_tmem + bcol + 4 * c, accumulate);
            else
              tc_mma_nvf4(acc, w_desc + (uint64_t)(2 * j), x_desc + (uint64_t)(2 * j), idesc0,
                          sfw_tmem + bcol + 4 * c, sfx_tmem + bcol + 4 * c, accumulate);
          }
        }
        tc_commit(bar(kEmpty + s));
        if (i == my_stages - 1) tc_commit(bar(kAccFull + (j & 1)));
      }
    }
    __syncwarp();
  }

  // -------------------------------------- partial sums -> owners -> output ---
  const bool epi = warp >= 2;
  const int q = warp & 3;
  const int wrow = q * 32 + lane;                 // weight row within the tile = accumulator lane
  float alpha = 1.0f;
  if (epi) {
    if (sp.after_producer) griddep_wait();         // alpha comes from the kernel before this one
    if (owner) alpha = load_alpha(p);
  }
  bool have_peers = true;
  for (int j = 0; j < my_tiles; ++j) {             // one pass unless persistent
    const int n_tile = tile0 + j * tile_stride;
    bool have_acc = false;
    float bias = 0.0f;
    if (epi && owner && p.bias && n_tile * 128 + wrow < p.n) {
      const int row = n_tile * 128 + wrow;
      if constexpr (sizeof(OutT) == 4) bias = __ldg(static_cast<const float*>(p.bias) + row);
      else if constexpr (std::is_same<OutT, __half>::value) bias = __half2float(static_cast<const __half*>(p.bias)[row]);
      else bias = __bfloat162float(static_cast<const __nv_bfloat16*>(p.bias)[row]);
    }
    if (epi && my_stages > 0) {
      have_acc = __all_sync(0xffffffffu, mbar_wait_bounded(bar(kAccFull + (j & 1)), (uint32_t)(j >> 1) & 1u, abort_flag));
      if (!have_acc) {
        *abort_flag = 1;
        if (lane == 0) atomicOr(p.status, kErrEpilogue);
      }
      tc_fence_after_sync();
    }
    const uint32_t t_row = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(j & 1) * kAccBufCols;
    if (sp.split > 1) {
      // A rank whose receive buffer lies in its stage area is ready only now: its epilogue warps arrive after its
      // last MMA has completed (all TMA writes landed, all MMA reads done).
      if (!sp.recv_behind_ring) cluster_arrive();
      cluster_wait();
      if (epi) {
        // This rank's partial for every owner but itself -> its own (drained) stage area, one block
        // [128 rows][tok + 4] per owner, then one bulk copy per warp and owner into that owner's receive buffer;
        // slot of sender r at owner o: r for r < o, r - 1 above.
        for (int o = 0; o < sp.owners; ++o) {
          if (o == (int)rank) continue;
          const uint32_t block = stage_base + (uint32_t)o * block_bytes;
          const uint32_t stage_row = block + (uint32_t)wrow * ld * 4u;
          for (int c = 0; c < sp.tok; c += 16) {
            uint32_t r[16];
            if (have_acc) {
              tmem_ld_32x32b_x16(t_row + o * sp.tok + c, r);
              tmem_ld_wait();
            } else {
#pragma unroll
              for (int t = 0; t < 16; ++t) r[t] = 0u;
            }
#pragma unroll
            for (int v = 0; v < 4; ++v)
              st_shared_v4(stage_row + (uint32_t)(c + 4 * v) * 4u,
                           make_uint4(r[4 * v], r[4 * v + 1], r[4 * v + 2], r[4 * v + 3]));
          }
        }
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) {
          const uint32_t warp_bytes = 32u * ld * 4u, warp_off = (uint32_t)q * warp_bytes;
          for (int o = 0; o < sp.owners; ++o) {
            if (o == (int)rank) continue;
            const uint32_t slot = (int)rank < o ? rank : rank - 1u;
            bulk_copy_to_cta(map_to_cta(smem_u32(recv_buf), (uint32_t)o) + slot * block_bytes + warp_off,
                             stage_base + (uint32_t)o * block_bytes + warp_off, warp_bytes,
                             map_to_cta(bar(kReduce), (uint32_t)o));
          }
        }
        __syncwarp();
      }
      if (epi && owner) {
        have_peers = __all_sync(0xffffffffu, mbar_wait_bounded(bar(kReduce), 0, abort_flag));
        if (!have_peers) {
          *abort_flag = 1;
          if (lane == 0) atomicOr(p.status, kErrEpilogue);
        }
      }
      // Second phase: a rank may leave only after every owner has received every copy (the copies' source is the
      // sender's shared memory); an owner arrives here once it has its data and adds while the others wait.  Nothing
      // written before this arrival is read by another CTA afterwards, so it needs no release.
      cluster_arrive_relaxed();
    }
    if (epi && owner) {
      OutT* d = static_cast<OutT*>(p.d);
      // staging tile [16 tokens][128 columns]: in the drained stage area, behind the blocks staged for sending, or
      // (persistent) behind the ring
      OutT* out_tile = reinterpret_cast<OutT*>(smem + sp.out_tile_offset);
      const int tok0 = (int)rank * sp.tok;
      const bool fused = p.act != 0 || p.out_gs != nullptr;            // 16-bit value types only
      const int tile_w = p.act ? 64 : 128;                              // output columns this tile of 128 weight rows yields
      const float out_gs = p.out_gs ? __ldg(p.out_gs) : 1.0f, rcp_out_gs = rcp_approx_ftz(out_gs), rcp6 = rcp_approx_ftz(6.0f);
      for (int c = 0; c < sp.tok; c += 16) {
        uint32_t r[16];
        if (have_acc) {
          tmem_ld_32x32b_x16(t_row + tok0 + c, r);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int t = 0; t < 16; ++t) r[t] = 0u;
        }
        float part[16];
#pragma unroll
        for (int t = 0; t < 16; ++t) part[t] = __uint_as_float(r[t]);
        if (have_peers) {
          for (int pr = 0; pr < sp.split - 1; ++pr) {
            const float4* src = reinterpret_cast<const float4*>(recv_buf + (pr * 128 + wrow) * ld + c);
#pragma unroll
            for (int v = 0; v < 4; ++v) {
              const float4 f = src[v];
              part[4 * v] += f.x; part[4 * v + 1] += f.y; part[4 * v + 2] += f.z; part[4 * v + 3] += f.w;
            }
          }
        }
        // Transpose through shared memory: this thread holds 16 tokens of one output column, the output rows are
        // tokens.  Writing them as they are costs 16 two-byte stores per thread; staged, a thread stores 16 bytes.
        if (c != 0 || j != 0) named_barrier_sync(1, 128);  // the previous chunk has left the staging tile
        if constexpr (sizeof(OutT) == 2) {
          if (fused) {
            // Gated activation: the 32 weight rows of this warp are 16 gate rows and their 16 up rows, so lane l < 16
            // finds its up value in lane l + 16 and the warp yields 16 output columns.  Then (or instead) the staged
            // tile is quantized to NVFP4 block by block, each block by one thread, with the quantizer's own function.
#pragma unroll
            for (int t = 0; t < 16; ++t) {
              float v = fmaf(part[t], alpha, bias);
              if constexpr (std::is_same<OutT, __half>::value) v = __half2float(__float2half_rn(v));
              else v = __bfloat162float(__float2bfloat16_rn(v));
              if (p.act) {
                const float up = __shfl_down_sync(0xffffffffu, v, 16);
                v = silu_mul_16bit<OutT>(v, up);
              }
              if (!p.act || lane < 16) {
                const int oc = p.act ? q * 16 + lane : wrow;
                if constexpr (std::is_same<OutT, __half>::value) out_tile[t * tile_w + oc] = __float2half_rn(v);
                else out_tile[t * tile_w + oc] = __float2bfloat16_rn(v);
              }
            }
            named_barrier_sync(1, 128);
            const int out_cols = p.act ? p.n / 2 : p.n;
            if (p.out_gs == nullptr) {
              const int segs = tile_w / 8;                   // 16-byte segments per token row of the tile
              for (int sidx = (int)threadIdx.x - 64; sidx < 16 * segs; sidx += 128) {
                const int t = sidx / segs, seg = sidx % segs;
                const int token = tok0 + c + t, col = n_tile * tile_w + seg * 8;
                if (token < p.m && col < out_cols)
                  *reinterpret_cast<uint4*>(d + (int64_t)token * out_cols + col) =
                      *reinterpret_cast<const uint4*>(out_tile + t * tile_w + seg * 8);
              }
            } else {
              using V2 = typename Vec2<OutT>::type;
              const int nblk = tile_w / 16, k_tiles = (out_cols + 63) / 64;
              uint8_t* out_fp4 = static_cast<uint8_t*>(p.d);
              for (int e = (int)threadIdx.x - 64; e < 16 * nblk; e += 128) {
                const int t = e / nblk, b = e % nblk;
                const int token = tok0 + c + t, ocol = n_tile * tile_w + b * 16;
                const uint4* src = reinterpret_cast<const uint4*>(out_tile + t * tile_w + b * 16);
                const uint4 lo = src[0], hi = src[1];
                const uint32_t w[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
                V2 h2[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) h2[i] = *reinterpret_cast<const V2*>(&w[i]);
                uint8_t sf;
                const uint2 qv = nvfp4_quantize_block<OutT>(h2, out_gs, rcp_out_gs, rcp6, sf);
                if (token < p.m && ocol < out_cols)
                  *reinterpret_cast<uint2*>(out_fp4 + (int64_t)token * (out_cols / 2) + ocol / 2) = qv;
                if (ocol / 64 < k_tiles)      // token < 128: rows [m, nt) of the one 128-row scale tile get zero scales
                  p.out_sf[(int64_t)(ocol / 64) * 512 + (token % 32) * 16 + (token / 32) * 4 + (ocol % 64) / 16] =
                      (token < p.m && ocol < out_cols) ? sf : (uint8_t)0;      // padding stays zero under a NaN scale too
              }
            }
            continue;
          }
        }
#pragma unroll
        for (int t = 0; t < 16; ++t) {
          const float v = fmaf(part[t], alpha, bias);
          if constexpr (sizeof(OutT) == 4) out_tile[t * 128 + wrow] = v;
          else if constexpr (std::is_same<OutT, __half>::value) out_tile[t * 128 + wrow] = __float2half_rn(v);
          else out_tile[t * 128 + wrow] = __float2bfloat16_rn(v);
        }
        named_barrier_sync(1, 128);
        constexpr int kSegs = 128 * (int)sizeof(OutT) / 16;   // 16-byte segments per token row
        constexpr int kSegElems = 16 / (int)sizeof(OutT);
        for (int sidx = (int)threadIdx.x - 64; sidx < 16 * kSegs; sidx += 128) {
          const int t = sidx / kSegs, seg = sidx % kSegs;
          const int token = tok0 + c + t, col = n_tile * 128 + seg * kSegElems;
          if (token < p.m && col < p.n)
            *reinterpret_cast<uint4*>(d + (int64_t)token * p.n + col) =
                *reinterpret_cast<const uint4*>(out_tile + t * 128 + seg * kSegElems);
        }
      }
      // NVFP4 output: the scale rows between the padded token count and 128 are zero in the quantizer's output too
      if constexpr (sizeof(OutT) == 2) {
        if (fused && p.out_gs != nullptr && rank == 0) {
          const int out_cols = p.act ? p.n / 2 : p.n;
          const int nblk = tile_w / 16, k_tiles = (out_cols + 63) / 64;
          for (int e = (int)threadIdx.x - 64; e < (128 - sp.nt) * nblk; e += 128) {
            const int row = sp.nt + e / nblk, ocol = n_tile * tile_w + (e % nblk) * 16;
            if (ocol / 64 < k_tiles)
              p.out_sf[(int64_t)(ocol / 64) * 512 + (row % 32) * 16 + (row / 32) * 4 + (ocol % 64) / 16] = (uint8_t)0;
          }
        }
      }
    }
    if (epi && sp.persistent) {
      // this tile's accumulator is in registers or stored: the issuer may overwrite it two tiles on
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(kAccEmpty + (j & 1)));
    }
  }  // tiles
  if (sp.split > 1) cluster_wait();
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  if (warp == 1) tmem_dealloc(tmem_base, kSkinnyTmemCols);
}

// K split for n_tiles weight tiles: double the cluster while all CTAs still run in one wave and every rank keeps
// at least 2048 elements of K, about what the exchange of partial sums costs.  Measured on B200 (cold L2, events):
// K = 14336, N = 4096: 16 tokens 20 / 15.5 / 12.6 us with 1 / 2 / 4 ranks; 128 tokens 29.6 / 23.6 / 21.5 us (the
// 128-row tile kernel: 33.6 us); at K = 4096 a second rank gains about 1 us and more ranks nothing.
inline int skinny_split(int n_tiles, int64_t k, int sm_count) {
  int split = 1;
  while (split < kSkinnyMaxSplit && n_tiles * split * 2 <= sm_count && k >= (int64_t)split * 2 * 2048) split *= 2;
  return split;
}

// Shapes this kernel is the better choice for: up to 32 tokens always; up to 64 unless the weight tiles alone need
// more than one wave of CTAs (the tokens then fill half of a 128-row tile anyway); up to 128 while the weight tiles
// leave at least half of the SMs idle, so that splitting K can use them.
inline bool skinny_preferred(int64_t m, int64_t n, int sm_count) {
  if (m > kSkinnyMaxTokens) return false;
  const int64_t n_tiles = ceil_div(n, 128);
  if (m > 64) return n_tiles * 2 <= sm_count;
  return m <= 32 || n_tiles <= sm_count;
}

template <bool MX, typename OutT, int BOXES>
int launch_skinny_boxes(const GemmParams& base, const void* a, const void* b, int sm_count, cudaStream_t stream,
                        bool after_producer) {
  using C = SkinnyCfg<MX, BOXES>;
  constexpr int kMaxTokens = BOXES == 4 ? 64 : 128;
  SkinnyParams sp{};
  sp.g = base;
  sp.after_producer = after_producer ? 1 : 0;
  const int m = base.m, n = base.n, k = base.k;
  const int n_tiles = (int)ceil_div(n, 128);
  const int total_stages = (int)ceil_div(k, C::kStageElems);
  const uint32_t budget = (uint32_t)kSmemLimit - 2048u;
  int split = skinny_split(n_tiles, k, sm_count);
  uint32_t smem_bytes = 0;
  unsigned grid = 0;
  // More tiles than SMs: every CTA takes the same number of tiles (448 tiles on 148 SMs: 112 CTAs with 4 each, not
  // three full waves and a fourth of 4 CTAs) and streams through them without draining its ring in between.
  const bool persistent = m <= 32 && n_tiles > sm_count;
  if (persistent) {
    const int rounds = (int)ceil_div(n_tiles, sm_count);
    grid = (unsigned)ceil_div(n_tiles, rounds);
    sp.persistent = 1;
    sp.nt = sp.tok = (int)round_up(m, 16);
    sp.split = sp.owners = split = 1;
    sp.stage_bytes = (uint32_t)round_up(BOXES * (C::kWBoxBytes + (uint32_t)sp.nt * kStageKBytes) + 2 * C::kSfBytes, 1024);
    const int max_stages = (int)((budget - kSkinnyOutTileBytes) / sp.stage_bytes);
    NVFP_REQUIRE(max_stages >= 1, "internal: a stage of %u bytes does not fit shared memory", sp.stage_bytes);
    sp.stages_per_rank = total_stages;
    sp.num_stages = std::max(1, std::min(total_stages * rounds, max_stages));
    const uint32_t ring_bytes = (uint32_t)sp.num_stages * sp.stage_bytes;
    sp.out_tile_offset = sp.recv_offset = ring_bytes;
    sp.recv_behind_ring = 1;
    sp.bars_offset = ring_bytes + kSkinnyOutTileBytes;
    smem_bytes = sp.bars_offset + 2048;
  }
  for (; !persistent; split /= 2) {
    // Every rank an owner when each can have a multiple of 16 tokens without padding the MMA beyond its limit and
    // there is more than one chunk of tokens to share out; else the leader alone, which is only worth it for one
    // chunk of tokens (32 and more tokens into one CTA cost more than the split saves).
    int nt = (int)round_up(m, 16), owners = 1;
    const int nt_scatter = (int)round_up(m, 16 * split);
    const bool scatter = split > 1 && nt >= 32 && nt_scatter <= kMaxTokens;
    if (split > 1 && nt >= 32 && !scatter) continue;
    if (scatter) {
      nt = nt_scatter;
      owners = split;
    }
    sp.nt = nt;
    sp.split = split;
    sp.owners = owners;
    sp.tok = nt / owners;
    sp.stage_bytes = (uint32_t)round_up(BOXES * (C::kWBoxBytes + (uint32_t)nt * kStageKBytes) + 2 * C::kSfBytes, 1024);
    const int max_stages = (int)(budget / sp.stage_bytes);
    NVFP_REQUIRE(max_stages >= 1, "internal: a stage of %u bytes does not fit shared memory", sp.stage_bytes);
    sp.stages_per_rank = (int)ceil_div(total_stages, split);
    sp.num_stages = std::max(1, std::min(sp.stages_per_rank, max_stages));
    const uint32_t ring_bytes = (uint32_t)sp.num_stages * sp.stage_bytes;
    const uint32_t block_bytes = skinny_block_bytes(sp.tok);
    const uint32_t staging_bytes = split > 1 ? (uint32_t)owners * block_bytes : 0u;
    const uint32_t recv_bytes = (uint32_t)(split - 1) * block_bytes;
    sp.out_tile_offset = staging_bytes;
    if (ring_bytes + recv_bytes <= budget && staging_bytes + kSkinnyOutTileBytes <= ring_bytes) {
      sp.recv_behind_ring = 1;
      sp.recv_offset = ring_bytes;
      sp.bars_offset = ring_bytes + recv_bytes;
      smem_bytes = ring_bytes + recv_bytes + 2048;
      break;
    }
    if (staging_bytes + kSkinnyOutTileBytes + recv_bytes <= ring_bytes) {
      sp.recv_behind_ring = 0;
      sp.recv_offset = staging_bytes + kSkinnyOutTileBytes;
      sp.bars_offset = ring_bytes;
      smem_bytes = ring_bytes + 2048;
      break;
    }
    NVFP_REQUIRE(split > 1, "internal: the epilogue's buffers do not fit %u bytes of stages", ring_bytes);
  }
  CUtensorMap map_w, map_x;
  if (int rc = make_operand_map(&map_w, b, n, k, 128)) return rc;
  if (int rc = make_operand_map(&map_x, a, m, k, sp.nt)) return rc;
  auto kernel = fp4_gemm_skinny_kernel<MX, OutT, BOXES>;
  if (int rc = ensure_dynamic_smem(kernel, (int)smem_bytes)) return rc;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(persistent ? grid : (unsigned)(n_tiles * sp.split));
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = smem_bytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  int num_attrs = 0;
  if (sp.split > 1) {
    attr[num_attrs].id = cudaLaunchAttributeClusterDimension;
    attr[num_attrs].val.clusterDim.x = (unsigned)sp.split;
    attr[num_attrs].val.clusterDim.y = 1;
    attr[num_attrs].val.clusterDim.z = 1;
    ++num_attrs;
  }
  if (after_producer) {
    attr[num_attrs].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[num_attrs].val.programmaticStreamSerializationAllowed = 1;
    ++num_attrs;
  }
  cfg.attrs = attr;
  cfg.numAttrs = num_attrs;
  NVFP_CUDA(cudaLaunchKernelEx(&cfg, kernel, map_w, map_x, sp));
  return NVFP_OK;
}

// Up to 64 tokens: stages of 1024 elements of K; above, the activation box is as large as the weight box and
// stages of 512 keep three of them in shared memory.  Smaller stages for the decode shapes (256 or 512 elements, so
// that the first MMAs start before a whole 88 KB stage has landed) measured slower or equal on every one of them.
template <bool MX, typename OutT>
int launch_skinny(const GemmParams& base, const void* a, const void* b, int sm_count, cudaStream_t stream,
                  bool after_producer = false) {
  if (base.m <= 64) return launch_skinny_boxes<MX, OutT, 4>(base, a, b, sm_count, stream, after_producer);
  return launch_skinny_boxes<MX, OutT, 2>(base, a, b, sm_count, stream, after_producer);
}
