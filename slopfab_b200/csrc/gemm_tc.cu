// tcgen05 GEMMs of the quantized Linear:  y[M,N] = epilogue( A[M,K] * W[N,K]^T ).
//
// One persistent, warp-specialised kernel template serves three operand kinds:
//   kI8    int8 activations x int8 weights -> int32 (W4A8 / W6A8 after expansion;
//          replaces the cuBLAS int8 GemmEx + output_bf16 + add_bias launches of
//          the reference, src/cuda/linear.cu:202-206)
//   kNvfp4 packed e2m1 x e2m1 with one ue4m3 scale per 16 elements -> fp32
//          (replaces nvfp4_gemm_kernel, src/cuda/nvfp4_gemm.cu:346-485)
//   kBf16  bf16 x bf16 -> fp32 (the dequantize-then-GEMM arm, src/cuda/linear.cu:243-246)
//
// Layout of the work: a CTA owns one SM and walks output tiles of 128 x BN.
// Warp 0 (one lane) streams K-slabs of 128 bytes per row into a ring of shared
// memory stages with TMA (128-byte swizzle, no multicast). Warp 1 (one lane)
// issues tcgen05.mma from shared-memory descriptors into a TMEM accumulator;
// a commit releases each stage back to the producer. Warps 4-11 drain a finished
// accumulator with tcgen05.ld, apply the fused epilogue and store bf16, while
// the MMA warp already fills the other accumulator buffer. Warps 12-15 (nvfp4)
// copy block scales from shared memory into TMEM, one warp per 64-element k-block.
// The four warpgroups rebalance registers with setmaxnreg: the single-lane roles
// give theirs up so that an epilogue thread can hold its whole slice of a tile.
//
// Every wait is bounded: a barrier that does not complete within kWaitCycles
// makes the waiting thread record a code in the status word, raise the CTA's
// abort flag and fall through to the common exit, where the producer waits
// (bounded) for its own copies in flight and TMEM is released.
#include "gemm_common.cuh"

namespace sfq {
namespace {

template <int KIND, int BN, int ACC> struct Cfg {
  static constexpr int kStageA = kBM * kSlabBytes;
  static constexpr int kStageB = BN * kSlabBytes;
  // nvfp4: per stage 4 k-blocks of 64 elements; one 512-byte scale atom per (128 rows, k-block)
  static constexpr int kStageSfa = KIND == kNvfp4 ? 4 * 512 : 0;
  static constexpr int kStageSfb = KIND == kNvfp4 ? (BN / 128) * 4 * 512 : 0;
  static constexpr int kStageBytes = kStageA + kStageB + kStageSfa + kStageSfb;
  static constexpr int kBarrierBytes = 5120;   // barriers + the epilogue's column operands
  static constexpr int kStagingBytes = 8 * 2048;  // one 32x32 bf16 transpose block per epilogue warp
  static constexpr int kRingBudget = 227 * 1024 - 1024 - kBarrierBytes - kStagingBytes;
  static constexpr int kStages = kRingBudget / kStageBytes > 8 ? 8 : kRingBudget / kStageBytes;
  static constexpr int kAccCols = BN * ACC;
  static constexpr int kSfSlotCols = KIND == kNvfp4 ? 4 * 4 + 4 * (BN / 32) : 0;  // SFA 4 cols, SFB BN/32 cols per k-block
  static constexpr int kTmemCols = 512;
  static constexpr int kSmemBytes = kStages * kStageBytes + kBarrierBytes + kStagingBytes + 1024;  // +1024 alignment slack
  // one TMEM scale slot per shared-memory stage, so a stage and its scales are released together
  static_assert(kAccCols + kStages * kSfSlotCols <= 512, "TMEM budget");
  static_assert(kStages >= 2, "pipeline needs at least two stages");
};

template <int KIND, int BN, int ACC, bool GATED>
__global__ void __launch_bounds__(kThreads, 1)
gemm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, GemmArgs g) {
  using C = Cfg<KIND, BN, ACC>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  Shared* sh = reinterpret_cast<Shared*>(smem + C::kStages * C::kStageBytes);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int tiles_m = (g.M + kBM - 1) / kBM;
  const int tiles_n = (g.N + BN - 1) / BN;
  const int num_tiles = tiles_m * tiles_n;
  const int row_bytes = KIND == kNvfp4 ? g.K / 2 : (KIND == kBf16 ? g.K * 2 : g.K);
  const int k_stages = (row_bytes + kSlabBytes - 1) / kSlabBytes;
  const int band = g.band_m > 0 ? g.band_m : 16;  // m-tiles per raster band

  auto tile_coords = [&](int t, int& tm, int& tn) {
    // Bands of `band` row-tiles sweep all column tiles, row-tile fastest inside
    // a band, so one wave of CTAs shares a few weight slabs and a few activation slabs in L2.
    const int per_band = band * tiles_n;
    const int b = t / per_band;
    const int r = t - b * per_band;
    const int rows_in_band = min(band, tiles_m - b * band);
    tn = r / rows_in_band;
    tm = b * band + (r - tn * rows_in_band);
  };

  if (threadIdx.x == 0) {
    for (int s = 0; s < C::kStages; ++s) {
      mbar_init(smem_u32(&sh->full[s]), 1);
      mbar_init(smem_u32(&sh->empty[s]), 1);
    }
    for (int a = 0; a < ACC; ++a) {
      mbar_init(smem_u32(&sh->acc_full[a]), 1);
      mbar_init(smem_u32(&sh->acc_empty[a]), 8);
    }
    for (int i = 0; i < C::kStages; ++i) mbar_init(smem_u32(&sh->sf_full[i]), 4);
    sh->abort = 0;
    sh->wait_cycles = g.wait_cycles > 0 ? g.wait_cycles : kWaitCycles;
    fence_barrier_init();
    prefetch_tensormap(&map_a);
    prefetch_tensormap(&map_b);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(&sh->tmem_base), C::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = sh->tmem_base;

  // Each role's code sits directly under its warpgroup's setmaxnreg, so the compiler budgets it accordingly.
  //
  // The producer, MMA and scale-copy roles run as CONVERGED warps: all 32 lanes walk the loop and poll the
  // barriers, and one elected lane issues the asynchronous instructions. A lone lane inside a divergent branch
  // measured ~80 cycles per tcgen05 instruction (its operands are moved into uniform registers one by one);
  // from a converged warp the same instruction issues in ~50, which is what lets one warp keep the tensor
  // pipe fed (4 MMAs + 1 commit + 1 wait per 512-cycle stage).
  if (warp < 4) {
    reg_dec<kRegsLean>();
    if (warp == 0) {
      // ------------------------------------------------------------ producer
      uint32_t it = 0;  // running stage counter
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        int tm, tn;
        tile_coords(t, tm, tn);
        for (int ks = 0; ks < k_stages; ++ks, ++it) {
          const int s = it % C::kStages;  // kStages is a compile-time constant
          const uint32_t ph = (it / C::kStages) & 1;
          if (!(ok = wait_barrier_warp(smem_u32(&sh->empty[s]), ph ^ 1, sh, g.status, 1))) break;
          if (elect_one()) {
            uint8_t* stage = smem + s * C::kStageBytes;
            const uint32_t bar = smem_u32(&sh->full[s]);
            uint32_t bytes = C::kStageA + C::kStageB;
            int kb_valid = 4, tiles_b = 0;
            if constexpr (KIND == kNvfp4) {
              kb_valid = min(4, (row_bytes - ks * kSlabBytes) / kMmaKBytes);
              tiles_b = min(BN / 128, (g.N - tn * BN + 127) / 128);
              bytes += (1 + tiles_b) * kb_valid * 512;
            }
            mbar_arrive_expect_tx(bar, bytes);
            if (int(it) == g.test_drop_iteration) bytes = 0;  // test hook: the bytes were announced, the loads are left out
            if (bytes != 0) tma_load_2d(smem_u32(stage), &map_a, ks * kSlabBytes, tm * kBM, bar);
            if (bytes != 0) tma_load_2d(smem_u32(stage + C::kStageA), &map_b, ks * kSlabBytes, tn * BN, bar);
            if (KIND == kNvfp4 && bytes != 0) {
              const int k_tiles = g.K / 64;  // scale atoms per 128-row tile
              const uint8_t* sfa = g.a_scale_tiled + (size_t(tm) * k_tiles + size_t(ks) * 4) * 512;
              bulk_load(smem_u32(stage + C::kStageA + C::kStageB), sfa, kb_valid * 512, bar);
              for (int rt = 0; rt < tiles_b; ++rt) {
                const uint8_t* sfb = g.w_scale_tiled + (size_t(tn * (BN / 128) + rt) * k_tiles + size_t(ks) * 4) * 512;
                bulk_load(smem_u32(stage + C::kStageA + C::kStageB + C::kStageSfa + rt * 4 * 512), sfb, kb_valid * 512,
                          bar);
              }
            }
          }
          __syncwarp();
        }
      }
      if (!ok && lane == 0) {
        // Aborting: let copies already in flight land before the CTA's shared memory is released.
        const long long start = clock_now();
        for (uint32_t back = 1; back <= uint32_t(C::kStages) && back <= it; ++back) {
          const uint32_t j = it - back;
          const uint32_t bar = smem_u32(&sh->full[j % C::kStages]);
          while (!mbar_try_wait(bar, (j / C::kStages) & 1) && clock_now() - start < sh->wait_cycles / 4) {
          }
        }
      }
    } else if (warp == 1) {
      // ------------------------------------------------------------ MMA issuer
      constexpr uint32_t idesc = KIND == kI8 ? idesc_i8(kBM, BN) : (KIND == kNvfp4 ? idesc_nvfp4(kBM, BN) : idesc_bf16(kBM, BN));
      // Everything between two MMAs is serial latency on the tensor pipe's critical path. So: running
      // counters instead of divisions, descriptor low words derived by one add per stage, one barrier wait and
      // one commit per stage.
      bool ok = true;
      const uint32_t a_base = smem_u32(smem) >> 4;                       // start-address fields, 16-byte units
      const uint32_t b_base = smem_u32(smem + C::kStageA) >> 4;
      constexpr uint32_t kStageStep = C::kStageBytes >> 4;
      constexpr uint64_t kDescHi = (uint64_t(1024 >> 4) << 32) | (uint64_t(1) << 46) | (uint64_t(2) << 61);
      const int last_valid = min(4, (row_bytes - (k_stages - 1) * kSlabBytes + kMmaKBytes - 1) / kMmaKBytes);
      int s = 0;
      uint32_t ph = 0, tile_it = 0;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x, ++tile_it) {
        const int a = tile_it % ACC;
        if (!(ok = wait_barrier_warp(smem_u32(&sh->acc_empty[a]), ((tile_it / ACC) & 1) ^ 1, sh, g.status, 2))) break;
        tc_fence_after_sync();
        const uint32_t d = tmem + a * BN;
        for (int ks = 0; ks < k_stages; ++ks) {
          // nvfp4: the scale-copy warps arrive on sf_full[s] after they have seen full[s] themselves and their
          // copies into TMEM slot s have landed, so that one barrier stands for operands and scales alike.
          if constexpr (KIND == kNvfp4) {
            if (!(ok = wait_barrier_warp(smem_u32(&sh->sf_full[s]), ph, sh, g.status, 5))) break;
            tc_fence_after_sync();
          } else {
            if (!(ok = wait_barrier_warp(smem_u32(&sh->full[s]), ph, sh, g.status, 3))) break;
          }
          const uint64_t da = kDescHi | uint64_t(a_base + s * kStageStep);
          const uint64_t db = kDescHi | uint64_t(b_base + s * kStageStep);
          const int kb_valid = ks == k_stages - 1 ? last_valid : 4;
          const uint32_t sf_cols = tmem + C::kAccCols + s * C::kSfSlotCols;
          if (elect_one()) {
#pragma unroll
            for (int kb = 0; kb < 4; ++kb) {
              if (kb < kb_valid) {
                const uint32_t acc = (ks | kb) ? 1u : 0u;
                const uint64_t adv = uint64_t(kb * (kMmaKBytes >> 4));
                if constexpr (KIND == kI8)
                  mma_i8(d, da + adv, db + adv, idesc, acc);
                else if constexpr (KIND == kBf16)
                  mma_f16(d, da + adv, db + adv, idesc, acc);
                else
                  mma_nvfp4(d, da + adv, db + adv, idesc, acc, sf_cols + kb * 4, sf_cols + 16 + kb * (BN / 32));
              }
            }
            // One commit frees the stage's shared memory for the producer and its scale slot for the copy warps.
            tc_commit(smem_u32(&sh->empty[s]));
            if (ks == k_stages - 1) tc_commit(smem_u32(&sh->acc_full[a]));
          }
          __syncwarp();
          if (++s == C::kStages) s = 0, ph ^= 1;
        }
      }
    }
  } else if (warp >= 12) {
    reg_dec<kRegsLean>();
    // ------------------------------------------------------------ scale-factor copies (nvfp4 only)
    // Warp 12+kb handles k-block kb of every stage: shared memory -> TMEM slot s with one 32x128b copy per
    // (128-row tile, k-block), then a commit that arrives on sf_full[s] when they have landed. A slot is free
    // again when the MMAs that read it have completed, which is what empty[s] says.
    if constexpr (KIND == kNvfp4) {
      const int kb = warp - 12;
      constexpr uint64_t kSfHi = (uint64_t(128 >> 4) << 32) | (uint64_t(1) << 46);
      constexpr uint32_t kStageStep = C::kStageBytes >> 4;
      const uint32_t sfa0 = (smem_u32(smem) + C::kStageA + C::kStageB) >> 4;
      const int last_valid = min(4, (row_bytes - (k_stages - 1) * kSlabBytes + kMmaKBytes - 1) / kMmaKBytes);
      int s = 0;
      uint32_t ph = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        for (int ks = 0; ks < k_stages; ++ks) {
          // full[s] of this round completes only after the producer has seen empty[s] of the previous round, so the
          // loads having landed also says that the MMAs which read this stage's scale slot are done: one wait, not two
          if (!(ok = wait_barrier_warp(smem_u32(&sh->full[s]), ph, sh, g.status, 6))) break;
          tc_fence_after_sync();
          const int kb_valid = ks == k_stages - 1 ? last_valid : 4;
          const uint32_t sf_cols = tmem + C::kAccCols + s * C::kSfSlotCols;
          const uint32_t sfa = sfa0 + s * kStageStep;
          const uint32_t sfb = sfa + (C::kStageSfa >> 4);
          if (elect_one()) {
            if (kb < kb_valid) {
              tc_copy_32x128b_x4(sf_cols + kb * 4, kSfHi | uint64_t(sfa + kb * 32));
#pragma unroll
              for (int rt = 0; rt < BN / 128; ++rt)
                tc_copy_32x128b_x4(sf_cols + 16 + kb * (BN / 32) + rt * 4, kSfHi | uint64_t(sfb + (rt * 4 + kb) * 32));
            }
            tc_commit(smem_u32(&sh->sf_full[s]));
          }
          __syncwarp();
          if (++s == C::kStages) s = 0, ph ^= 1;
        }
      }
    }
  } else {
    reg_inc<kRegsEpilogue>();
    // ------------------------------------------------------------ epilogue (8 warps)
    // Warp w may only read TMEM lanes [32*(w%4), +32). Two warps share each lane quadrant and take alternate
    // 32-column chunks, so every scheduler holds two epilogue warps and their latencies overlap.
    const int quad = warp & 3;
    const int half = (warp - 4) >> 2;
    const int et = threadIdx.x - 128;  // 0..255 among the epilogue threads
    uint32_t tile_it = 0;
    bool ok = true;
    const bool vec_ok = (g.N % 8 == 0) && ((reinterpret_cast<uintptr_t>(g.y) & 15) == 0) && (g.ldy % 8 == 0);
    const bool has_bias = g.bias != nullptr;
    for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x, ++tile_it) {
      int tm, tn;
      tile_coords(t, tm, tn);
      const int a = tile_it % ACC;
      const uint32_t aph = (tile_it / ACC) & 1;
      // Per-column epilogue operands of this tile go to shared memory once (two buffers: the previous tile's
      // may still be in use by a slower warp until it reaches the named barrier below).
      float* cs_s = sh->col_scale[tile_it & 1];
      float* bs_s = sh->bias[tile_it & 1];
      if (et < BN) {
        const int col = tn * BN + et;
        float cs = g.global_scale, bs = 0.0f;
        if (col < g.N) {
          if constexpr (KIND == kI8) cs = __ldg(g.col_scale + col);
          if (has_bias)
            bs = g.bias_is_bf16 ? __bfloat162float(static_cast<const __nv_bfloat16*>(g.bias)[col])
                                : __ldg(static_cast<const float*>(g.bias) + col);
        }
        cs_s[et] = cs;
        bs_s[et] = bs;
      }
      if constexpr (GATED) {
        // Gated residual: the epilogue will read-modify-write this tile of y. Ask L2 for it now, a whole main loop
        // ahead, so those reads do not pay HBM latency on the store path (128 rows x BN bf16 = BN/64 lines per row).
        constexpr int kLinesPerRow = BN / 64;
        for (int l = et; l < kBM * kLinesPerRow; l += 256) {
          const int pr = tm * kBM + l / kLinesPerRow, pc = tn * BN + (l % kLinesPerRow) * 64;
          if (pr < g.M && pc < g.N) asm volatile("prefetch.global.L2 [%0];" ::"l"(g.y + size_t(pr) * g.ldy + pc));
        }
      }
      asm volatile("bar.sync 1, 256;" ::: "memory");
      if (!(ok = wait_barrier(smem_u32(&sh->acc_full[a]), aph, sh, g.status, 4))) break;
      tc_fence_after_sync();
      const int row = tm * kBM + quad * 32 + lane;
      const bool row_ok = row < g.M;
      const float rs = (KIND == kI8 && row_ok) ? __ldg(g.row_scale + row) : 1.0f;
      __nv_bfloat16* yrow = g.y + size_t(row_ok ? row : 0) * g.ldy;
      const int warp_row0 = tm * kBM + quad * 32;
      const int rows_ok = max(0, min(32, g.M - warp_row0));
      __nv_bfloat16* ywarp = g.y + size_t(min(warp_row0, g.M - 1)) * g.ldy;
      uint4* stage_w = reinterpret_cast<uint4*>(smem + C::kStages * C::kStageBytes + C::kBarrierBytes) + (warp - 4) * 128;
      // This warp takes the 32-column chunks half, half+2, ... of the tile. It first moves ALL of them from
      // TMEM into registers and hands the accumulator back to the MMA warp; arithmetic and stores follow, off
      // the tensor pipe's critical path.
      constexpr int kTileChunks = BN / 32;
      constexpr int kMaxJ = (kTileChunks + 1) / 2;
      const uint32_t tbase = tmem + a * BN + (uint32_t(quad * 32) << 16);
      int gate_idx[4] = {0, 0, 0, 0};
      const float* gate_row = nullptr;
      if constexpr (GATED) {
        gate_rows_for(g, warp_row0, lane, gate_idx);
        if (row_ok) gate_row = g.gate + size_t(__ldg(g.gate_index + row)) * g.N;
      }
      uint32_t r[kMaxJ][32];
#pragma unroll
      for (int j = 0; j < kMaxJ; ++j)
        if (half + 2 * j < kTileChunks) tmem_ld_32x32(tbase + (half + 2 * j) * 32, r[j]);
      tmem_ld_wait();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&sh->acc_empty[a]));
#pragma unroll
      for (int j = 0; j < kMaxJ; ++j) {
        const int c = half + 2 * j;
        const int col0 = tn * BN + c * 32;
        if (c >= kTileChunks || col0 >= g.N) continue;  // warp-uniform
        const int lc0 = c * 32;
        uint4 packed[4];
        if (!has_bias && g.act == SFQ_ACT_NONE)
          pack_chunk<KIND, false, false>(r[j], rs, cs_s + lc0, bs_s + lc0, packed);
        else if (g.act == SFQ_ACT_NONE)
          pack_chunk<KIND, true, false>(r[j], rs, cs_s + lc0, bs_s + lc0, packed);
        else
          pack_chunk<KIND, true, true>(r[j], rs, cs_s + lc0, bs_s + lc0, packed);
        if (vec_ok && col0 + 32 <= g.N) {
          if constexpr (GATED)
            flush_chunk(packed, stage_w, ywarp + col0, size_t(g.ldy), rows_ok, lane, g.gate + col0, size_t(g.N), gate_idx);
          else
            flush_chunk(packed, stage_w, ywarp + col0, size_t(g.ldy), rows_ok, lane);
        } else if (row_ok) {  // ragged N or unaligned output: element stores from this thread's own row
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            const uint32_t w4[4] = {packed[v].x, packed[v].y, packed[v].z, packed[v].w};
#pragma unroll
            for (int q = 0; q < 8; ++q) {
              const int col = col0 + v * 8 + q;
              if (col < g.N) {
                __nv_bfloat16 o = __ushort_as_bfloat16((unsigned short)((w4[q >> 1] >> (16 * (q & 1))) & 0xFFFFu));
                if (gate_row != nullptr)
                  o = __float2bfloat16(__fmaf_rn(__ldg(gate_row + col), __bfloat162float(o), __bfloat162float(yrow[col])));
                yrow[col] = o;
              }
            }
          }
        }
      }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem, C::kTmemCols);
  }
}

template <int KIND, int BN, int ACC, bool GATED>
void launch_epi(const void* a, const void* w, size_t row_bytes, const GemmArgs& g, cudaStream_t stream) {
  using C = Cfg<KIND, BN, ACC>;
  reserve_dynamic_smem(reinterpret_cast<const void*>(&gemm_kernel<KIND, BN, ACC, GATED>), C::kSmemBytes, "sfq gemm");
  const CUtensorMap ma = make_map(a, size_t(g.M), row_bytes, kBM);
  const CUtensorMap mb = make_map(w, size_t(g.N), row_bytes, BN);
  const int tiles = ((g.M + kBM - 1) / kBM) * ((g.N + BN - 1) / BN);
  const int grid = g.max_ctas > 0 ? std::min(tiles, g.max_ctas) : std::min(tiles, sm_count());
  gemm_kernel<KIND, BN, ACC, GATED><<<grid, kThreads, C::kSmemBytes, stream>>>(ma, mb, g);
  const cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) throw std::runtime_error(std::string("sfq gemm: launch failed: ") + cudaGetErrorString(e));
}

// The gated residual is a compile-time variant of the epilogue, so the plain store path carries none of its registers.
template <int KIND, int BN, int ACC>
void launch(const void* a, const void* w, size_t row_bytes, const GemmArgs& g, cudaStream_t stream) {
  if (g.gate != nullptr)
    launch_epi<KIND, BN, ACC, true>(a, w, row_bytes, g, stream);
  else
    launch_epi<KIND, BN, ACC, false>(a, w, row_bytes, g, stream);
}

}  // namespace

void gemm_int8(const int8_t* a, const int8_t* w, const GemmArgs& g, cudaStream_t stream) {
  if (g.M <= 0 || g.N <= 0) return;
  if (g.K <= 0 || g.K % 16 != 0) throw std::invalid_argument("sfq gemm int8: K must be a positive multiple of 16");
  if (!a || !w || !g.row_scale || !g.col_scale || !g.y || !g.status)
    throw std::invalid_argument("sfq gemm int8: null operand");
  // Default: CTA pairs on 256 x 256 tiles once there are at least two 128-row tiles to pair up. tile_n = 256 or
  // 128 selects the one-CTA kernel with that tile width (256 is the faster of the two at every DiT shape).
  if (g.act == SFQ_ACT_SWIGLU) {  // only the CTA-pair kernel pairs gate and up columns in one tile
    if (!gemm_pair_int8(a, w, g, stream)) throw std::runtime_error("sfq gemm int8: the SwiGLU epilogue needs the CTA-pair kernel, which this device cannot schedule");
    return;
  }
  if (g.tile_n == 0 && g.M > kBM && gemm_pair_int8(a, w, g, stream)) return;
  if (g.tile_n == 128)
    launch<kI8, 128, 2>(a, w, size_t(g.K), g, stream);
  else
    launch<kI8, 256, 2>(a, w, size_t(g.K), g, stream);
}

void gemm_nvfp4(const uint8_t* a, const uint8_t* w, const GemmArgs& g, cudaStream_t stream) {
  if (g.M <= 0 || g.N <= 0) return;
  if (g.K <= 0 || g.K % 64 != 0 || g.N % 128 != 0)
    throw std::invalid_argument("sfq gemm nvfp4: needs K % 64 == 0 and N % 128 == 0 (the scale tiling has no padded form)");
  if (!a || !w || !g.a_scale_tiled || !g.w_scale_tiled || !g.y || !g.status)
    throw std::invalid_argument("sfq gemm nvfp4: null operand");
  // One-CTA form: a 256-wide tile has one accumulator (256 columns + the scale slots); 128-wide tiles have two
  // but feed the tensor pipe less efficiently.
  if (g.act == SFQ_ACT_SWIGLU) {  // only the CTA-pair kernel pairs gate and up columns in one tile
    if (!gemm_pair_nvfp4(a, w, g, stream)) throw std::runtime_error("sfq gemm nvfp4: the SwiGLU epilogue needs the CTA-pair kernel, which this device cannot schedule");
    return;
  }
  if (g.tile_n == 0 && g.M > kBM && gemm_pair_nvfp4(a, w, g, stream)) return;
  if (g.tile_n == 128)
    launch<kNvfp4, 128, 2>(a, w, size_t(g.K) / 2, g, stream);
  else
    launch<kNvfp4, 256, 1>(a, w, size_t(g.K) / 2, g, stream);
}

void gemm_bf16(const __nv_bfloat16* a, const __nv_bfloat16* w, const GemmArgs& g, cudaStream_t stream) {
  if (g.M <= 0 || g.N <= 0) return;
  if (g.K <= 0 || g.K % 8 != 0) throw std::invalid_argument("sfq gemm bf16: K must be a positive multiple of 8");
  if (!a || !w || !g.y || !g.status) throw std::invalid_argument("sfq gemm bf16: null operand");
  if (g.act == SFQ_ACT_SWIGLU) {  // only the CTA-pair kernel pairs gate and up columns in one tile
    if (!gemm_pair_bf16(a, w, g, stream)) throw std::runtime_error("sfq gemm bf16: the SwiGLU epilogue needs the CTA-pair kernel, which this device cannot schedule");
    return;
  }
  if (g.tile_n == 0 && g.M > kBM && gemm_pair_bf16(a, w, g, stream)) return;
  if (g.tile_n == 128)
    launch<kBf16, 128, 2>(a, w, size_t(g.K) * 2, g, stream);
  else
    launch<kBf16, 256, 2>(a, w, size_t(g.K) * 2, g, stream);
}

}  // namespace sfq
