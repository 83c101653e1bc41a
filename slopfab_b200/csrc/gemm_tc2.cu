// CTA-pair form of the tcgen05 GEMMs (see gemm_tc.cu for the one-CTA form and the operand kinds).
//
// Two CTAs of a cluster share one 256 x 256 output tile: tcgen05.mma.cta_group::2 with M = 256. Each CTA
// streams ITS 128 rows of the activation and ITS 128 of the 256 weight rows of the tile (32 KB per 128-byte
// K-slab instead of 48 KB), and receives 128 x 256 of the result in its own TMEM. Per SM that is a third less
// shared-memory fill and L2 traffic for the same tensor work, and the smaller stages make the ring six deep
// (five for nvfp4) instead of four (three), which is what hides the load latency at K-slab granularity.
//
// Division of labour inside a pair:
//   both CTAs    warp 0 loads its own operand halves with TMA (no multicast); the bytes of BOTH CTAs are counted
//                on the leader's `full` barrier. Warps 4-11 drain the CTA's own accumulator and store its rows.
//   leader only  warp 1 issues the MMAs for the pair; its commits arrive on `empty` / `acc_full` in both CTAs.
//                For nvfp4 the same thread copies each k-block's scale atoms into TMEM of both CTAs (each from its own
//                shared memory) right in front of the MMA that reads them.
//   the peer's epilogue hands the accumulator back by arriving on the LEADER's acc_empty barrier.
// Tail of the persistent schedule: when the last wave would leave more than half of the pairs idle, its tiles are
// cut into two 256 x 128 halves (N = 128 MMAs, 64 weight rows per CTA), so that wave takes about two thirds of a
// full one instead of a whole one (config 2: 320 tiles over 74 pairs = 4 waves + 24 tiles -> 48 half tiles).
// Every wait is bounded as in the one-CTA kernel; both CTAs meet at a cluster barrier before TMEM is freed, so
// neither exits while its partner can still read its shared memory or signal its barriers.
#include "codec.cuh"
#include "gemm_common.cuh"

namespace sfq {
namespace {

constexpr int kPairBN = 256;
constexpr int kPairBM = 256;  // rows of a pair's tile, 128 per CTA

// W4 (int8 only): the weight arrives as W4A8 nibbles (64 bytes per row and K-slab) in a staging area of the stage and is
// expanded to int8 in the stage's B area by warps 12-15 (see the kernel).
template <int KIND, int ACC, bool W4 = false> struct PairCfg {
  static constexpr int kStageA = kBM * kSlabBytes;            // this CTA's 128 activation rows
  static constexpr int kStageB = (kPairBN / 2) * kSlabBytes;  // this CTA's 128 of the tile's 256 weight rows
  static constexpr int kStageSfa = KIND == kNvfp4 ? 4 * 512 : 0;      // scales of this CTA's rows, 4 k-blocks
  static constexpr int kStageSfb = KIND == kNvfp4 ? 2 * 4 * 512 : 0;  // scales of ALL 256 weight rows
  static constexpr int kStageW4 = W4 ? (kPairBN / 2) * (kSlabBytes / 2) : 0;  // this CTA's 128 weight rows as nibbles
  static constexpr int kStageBytes = kStageA + kStageB + kStageSfa + kStageSfb + kStageW4;
  static constexpr int kBarrierBytes = 5120;
  static constexpr int kStagingBytes = 8 * 2048;
  static constexpr int kRingBudget = 227 * 1024 - 1024 - kBarrierBytes - kStagingBytes;
  static constexpr int kStages = kRingBudget / kStageBytes > 8 ? 8 : kRingBudget / kStageBytes;
  static constexpr int kAccCols = kPairBN * ACC;
  static constexpr int kSfSlotCols = KIND == kNvfp4 ? 4 * 4 + 4 * (kPairBN / 32) : 0;
  static constexpr int kTmemCols = 512;
  static constexpr int kSmemBytes = kStages * kStageBytes + kBarrierBytes + kStagingBytes + 1024;
  // what both CTAs land per stage on the leader's barrier (TMA counts whole boxes); W4: the activations only, the
  // nibbles are counted on each CTA's own w4_full barrier
  static constexpr uint32_t kTxBytes = W4 ? 2u * kStageA : 2u * kStageBytes;
  static constexpr uint32_t kTxBytesNarrow = 2u * (kStageA + kStageB / 2 + kStageSfa + kStageSfb / 2);  // 256 x 128 tile
  static_assert(kAccCols + kStages * kSfSlotCols <= 512, "TMEM budget");
  static_assert(kStageBytes % 1024 == 0, "stage bases must keep the 1024-byte swizzle alignment");
  static_assert(sizeof(Shared) <= kBarrierBytes, "barrier block");
};

// EPI selects the epilogue variant at compile time, so the plain store path carries none of the others' registers or
// branches: 0 = scales / bias / GELU, 1 = + gated residual (read-modify-write of y), 2 = SwiGLU over [gate | up].
enum { kEpiPlain = 0, kEpiGated = 1, kEpiSwiglu = 2 };

// TAIL: the schedule ends with tiles cut into 128-column halves (see above); without it every tile is 256 wide at
// compile time.
template <int KIND, int ACC, int EPI, bool TAIL, bool W4 = false>
__global__ void __launch_bounds__(kThreads, 1)
gemm_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                 const __grid_constant__ CUtensorMap map_sfa, const __grid_constant__ CUtensorMap map_sfb,
                 const __grid_constant__ CUtensorMap map_b_narrow, const __grid_constant__ CUtensorMap map_sfb_narrow,
                 GemmArgs g) {
  static_assert(!W4 || (KIND == kI8 && !TAIL && EPI == kEpiPlain), "the in-kernel W4 expansion is built for the plain int8 kernel");
  using C = PairCfg<KIND, ACC, W4>;
  constexpr int BN = kPairBN;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  Shared* sh = reinterpret_cast<Shared*>(smem + C::kStages * C::kStageBytes);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();  // 0 = leader
  const int pair = blockIdx.x >> 1;
  const int num_pairs = gridDim.x >> 1;
  const int tiles_m = (g.M + kPairBM - 1) / kPairBM;
  // SwiGLU epilogue: the weight rows are [gate | up], `inner` each, and a tile pairs 128 gate columns (the leader's
  // weight rows) with the 128 up columns of the same outputs (the peer's), so both meet in one accumulator row.
  constexpr bool swiglu = EPI == kEpiSwiglu;
  const int inner = g.N / 2;
  const int tiles_n = swiglu ? inner / (BN / 2) : (g.N + BN - 1) / BN;
  const int num_tiles = tiles_m * tiles_n;
  const int row_bytes = KIND == kNvfp4 ? g.K / 2 : (KIND == kBf16 ? g.K * 2 : g.K);
  const int k_stages = (row_bytes + kSlabBytes - 1) / kSlabBytes;
  // Pair tiles (256 rows) per raster band. A band sweeps every column tile, so between two uses of a weight slab the L2
  // sees one band of output, one band of activations and the whole weight: two pair tiles keep that near 55 MB at the
  // widest DiT layer (N = 13824) and cut the DRAM re-reads of the weight (380 MB instead of 586 MB per launch at
  // 27900 x 5120 -> 13824, same duration); wider bands only move more of the weight through DRAM.
  const int band = g.band_m > 0 ? (g.band_m + 1) / 2 : 2;

  // Work items: the tiles in raster order, except that the last `tail_split` of them appear as two 128-column
  // halves each. Every role decodes an item the same way.
  const int first_split = TAIL ? num_tiles - g.tail_split : num_tiles;
  const int num_work = TAIL ? num_tiles + g.tail_split : num_tiles;
  auto work_item = [&](int w, int& tm, int& tn, int& n_off, int& n_cols) {
    int t = w;
    n_off = 0;
    n_cols = BN;
    if (TAIL && w >= first_split) {
      const int j = w - first_split;
      t = first_split + (j >> 1);
      n_off = (j & 1) * (BN / 2);
      n_cols = BN / 2;
    }
    const int per_band = band * tiles_n;
    const int b = t / per_band;
    const int r = t - b * per_band;
    const int rows_in_band = min(band, tiles_m - b * band);
    tn = r / rows_in_band;
    tm = b * band + (r - tn * rows_in_band);
  };

  if (threadIdx.x == 0) {
    for (int s = 0; s < C::kStages; ++s) {
      mbar_init(smem_u32(&sh->full[s]), 1);     // used in the leader: its producer's arrive + both CTAs' bytes
      mbar_init(smem_u32(&sh->empty[s]), 1);    // in each CTA: the pair's MMAs of that stage are done
      if constexpr (W4) {
        mbar_init(smem_u32(&sh->w4_full[s]), 1);  // in each CTA: its own nibbles of the stage have landed
        mbar_init(smem_u32(&sh->sf_full[s]), 2);  // leader: the expanding warp of each CTA has written the stage's int8 rows
      }
    }
    for (int a = 0; a < ACC; ++a) {
      mbar_init(smem_u32(&sh->acc_full[a]), 1);    // in each CTA
      mbar_init(smem_u32(&sh->acc_empty[a]), 16);  // leader: eight epilogue warps of each CTA
    }
    sh->abort = 0;
    sh->wait_cycles = g.wait_cycles > 0 ? g.wait_cycles : kWaitCycles;
    fence_barrier_init();
    prefetch_tensormap(&map_a);
    prefetch_tensormap(&map_b);
  }
  if (warp == 1) {
    tmem_alloc_pair(smem_u32(&sh->tmem_base), C::kTmemCols);
    tmem_relinquish_pair();
  }
  tc_fence_before_sync();
  cluster_sync_all();  // barriers of both CTAs are initialised before anyone signals them
  tc_fence_after_sync();
  const uint32_t tmem = sh->tmem_base;

  if (warp < 4) {
    reg_dec<kRegsLean>();
    if (warp == 0) {
      // ------------------------------------------------------------ producer (both CTAs)
      uint32_t it = 0;
      bool ok = true;
      for (int t = pair; t < num_work && ok; t += num_pairs) {
        int tm, tn, n_off, n_cols;
        work_item(t, tm, tn, n_off, n_cols);
        const bool narrow = TAIL && n_cols != BN;
        for (int ks = 0; ks < k_stages; ++ks, ++it) {
          const int s = it % C::kStages;
          const uint32_t ph = (it / C::kStages) & 1;
          if (!(ok = wait_barrier_warp(smem_u32(&sh->empty[s]), ph ^ 1, sh, g.status, 1))) break;
          if (elect_one()) {
            uint8_t* stage = smem + s * C::kStageBytes;
            const uint32_t bar = smem_u32(&sh->full[s]);  // the loads redirect it to the leader's copy
            if (rank == 0) mbar_arrive_expect_tx(bar, narrow ? C::kTxBytesNarrow : C::kTxBytes);
            if constexpr (W4) {  // this CTA's 128 weight rows of the slab as nibbles (the map is passed in map_b's place)
              mbar_arrive_expect_tx(smem_u32(&sh->w4_full[s]), C::kStageW4);
              tma_load_2d(smem_u32(stage + C::kStageA + C::kStageB), &map_b, ks * (kSlabBytes / 2), tn * BN + int(rank) * (BN / 2),
                          smem_u32(&sh->w4_full[s]));
              tma_load_2d_pair(smem_u32(stage), &map_a, ks * kSlabBytes, tm * kPairBM + int(rank) * kBM, bar);
            } else if (int(it) != g.test_drop_iteration) {  // test hook: that iteration announces its bytes and leaves the loads out
              tma_load_2d_pair(smem_u32(stage), &map_a, ks * kSlabBytes, tm * kPairBM + int(rank) * kBM, bar);
              if (swiglu)
                tma_load_2d_pair(smem_u32(stage + C::kStageA), &map_b, ks * kSlabBytes, tn * (BN / 2) + int(rank) * inner, bar);
              else if (!narrow)
                tma_load_2d_pair(smem_u32(stage + C::kStageA), &map_b, ks * kSlabBytes, tn * BN + int(rank) * (BN / 2), bar);
              else
                tma_load_2d_pair(smem_u32(stage + C::kStageA), &map_b_narrow, ks * kSlabBytes, tn * BN + n_off + int(rank) * (BN / 4),
                                 bar);
              if constexpr (KIND == kNvfp4) {
                // scale arrays as [128-row tile][K/64 atoms of 512 bytes], 8-byte elements: 256 elements = 4 atoms
                tma_load_2d_pair(smem_u32(stage + C::kStageA + C::kStageB), &map_sfa, ks * 256, tm * 2 + int(rank), bar);
                if (swiglu) {  // scales of the gate rows' tile and of the up rows' tile, one 128-row tile each
                  tma_load_2d_pair(smem_u32(stage + C::kStageA + C::kStageB + C::kStageSfa), &map_sfb_narrow, ks * 256, tn, bar);
                  tma_load_2d_pair(smem_u32(stage + C::kStageA + C::kStageB + C::kStageSfa + C::kStageSfb / 2), &map_sfb_narrow,
                                   ks * 256, inner / 128 + tn, bar);
                } else if (!narrow) {
                  tma_load_2d_pair(smem_u32(stage + C::kStageA + C::kStageB + C::kStageSfa), &map_sfb, ks * 256, tn * 2, bar);
                } else {
                  tma_load_2d_pair(smem_u32(stage + C::kStageA + C::kStageB + C::kStageSfa), &map_sfb_narrow, ks * 256,
                                   tn * 2 + n_off / 128, bar);
                }
              }
            }
          }
          __syncwarp();
        }
      }
      if (!ok) {
        // Aborting: this CTA's loads in flight are counted on the leader's barriers, so it cannot poll for them;
        // give them far more time than a load takes before the shared memory may be released.
        const long long start = clock_now();
        while (clock_now() - start < 4000000ll) {
        }
      }
    } else if (warp == 1 && rank == 0) {
      // ------------------------------------------------------------ MMA issuer (leader)
      constexpr uint32_t idesc_wide = KIND == kI8 ? idesc_i8(kPairBM, BN) : (KIND == kNvfp4 ? idesc_nvfp4(kPairBM, BN) : idesc_bf16(kPairBM, BN));
      constexpr uint32_t idesc_narrow =
          KIND == kI8 ? idesc_i8(kPairBM, BN / 2) : (KIND == kNvfp4 ? idesc_nvfp4(kPairBM, BN / 2) : idesc_bf16(kPairBM, BN / 2));
      bool ok = true;
      const uint32_t a_base = (smem_u32(smem) & 0x3FFFFu) >> 4;  // descriptor address fields: offset in the CTA's window
      const uint32_t b_base = (smem_u32(smem + C::kStageA) & 0x3FFFFu) >> 4;
      constexpr uint32_t kStageStep = C::kStageBytes >> 4;
      constexpr uint64_t kDescHi = (uint64_t(1024 >> 4) << 32) | (uint64_t(1) << 46) | (uint64_t(2) << 61);
      const int last_valid = min(4, (row_bytes - (k_stages - 1) * kSlabBytes + kMmaKBytes - 1) / kMmaKBytes);
      int s = 0;
      uint32_t ph = 0, tile_it = 0;
      // nvfp4: this thread also copies the stage's scale atoms shared memory -> TMEM, each k-block's three copies right in
      // front of the MMA that reads them (copy -> MMA from one thread execute in issue order). TMEM scale slot s belongs to
      // stage s: full[s] of this round follows empty[s] of the previous one, i.e. the MMAs that read the slot are done.
      // W4: the expanding warps of both CTAs arrive on sf_full[st] when the stage's int8 weight rows are in place; the
      // activations' full[st] has normally completed long before and is checked behind it.
      auto stage_bar = [&](int st) { return smem_u32(W4 ? &sh->sf_full[st] : &sh->full[st]); };
      constexpr uint64_t kSfHi = (uint64_t(128 >> 4) << 32) | (uint64_t(1) << 46);
      const uint32_t sfa0 = ((smem_u32(smem) & 0x3FFFFu) + C::kStageA + C::kStageB) >> 4;
      // The barrier of the NEXT stage is probed (without blocking) in the same breath as a stage's MMAs are issued, so
      // in steady state the blocking wait and its round trip never sit between two stages' MMAs.
      uint32_t ready = 0;
      for (int t = pair; t < num_work && ok; t += num_pairs, ++tile_it) {
        const int a = tile_it % ACC;
        if (!(ok = wait_barrier_warp(smem_u32(&sh->acc_empty[a]), ((tile_it / ACC) & 1) ^ 1, sh, g.status, 2))) break;
        tc_fence_after_sync();
        const uint32_t d = tmem + a * BN;
        const bool narrow = TAIL && t >= first_split;
        const uint32_t idesc = narrow ? idesc_narrow : idesc_wide;
        const uint32_t sfb_step = narrow ? BN / 64 : BN / 32;  // TMEM columns of the weight scales per k-block
        for (int ks = 0; ks < k_stages; ++ks) {
          if (!__all_sync(0xffffffffu, ready != 0)) {
            if (!(ok = wait_barrier_warp(stage_bar(s), ph, sh, g.status, 3))) break;
          }
          if constexpr (W4) {
            if (!(ok = wait_barrier_warp(smem_u32(&sh->full[s]), ph, sh, g.status, 7))) break;
          }
          tc_fence_after_sync();
          const int s_next = s + 1 == C::kStages ? 0 : s + 1;
          const uint32_t ph_next = s_next == 0 ? ph ^ 1 : ph;
          const uint64_t da = kDescHi | uint64_t(a_base + s * kStageStep);
          const uint64_t db = kDescHi | uint64_t(b_base + s * kStageStep);
          const int kb_valid = ks == k_stages - 1 ? last_valid : 4;
          const uint32_t sf_cols = tmem + C::kAccCols + s * C::kSfSlotCols;
          ready = 1;  // the lanes that issue nothing do not vote against
          if (elect_one()) {
            if (KIND == kNvfp4 && kb_valid == 4 && !narrow) {
              ready = stage4_pair_nvfp4_cp(d, da, db, idesc, ks ? 1u : 0u, sf_cols, kSfHi | uint64_t(sfa0 + s * kStageStep),
                                           smem_u32(&sh->empty[s]), stage_bar(s_next), ph_next);
            } else if (KIND != kNvfp4 && kb_valid == 4) {
              // commit: frees the stage in both CTAs
              ready = stage4_pair<int(KIND)>(d, da, db, idesc, ks ? 1u : 0u, sf_cols, sf_cols + 16, sfb_step, smem_u32(&sh->empty[s]),
                                             stage_bar(s_next), ph_next);
            } else {
              ready = mbar_test_wait(stage_bar(s_next), ph_next);
#pragma unroll
              for (int kb = 0; kb < 4; ++kb) {
                if (kb < kb_valid) {
                  const uint32_t acc = (ks | kb) ? 1u : 0u;
                  const uint64_t adv = uint64_t(kb * (kMmaKBytes >> 4));
                  if constexpr (KIND == kI8)
                    mma_i8_pair(d, da + adv, db + adv, idesc, acc);
                  else if constexpr (KIND == kBf16)
                    mma_f16_pair(d, da + adv, db + adv, idesc, acc);
                  else {
                    const uint32_t sfa = sfa0 + s * kStageStep, sfb = sfa + (C::kStageSfa >> 4);
                    tc_copy_32x128b_x4_pair(sf_cols + kb * 4, kSfHi | uint64_t(sfa + kb * 32));
                    tc_copy_32x128b_x4_pair(sf_cols + 16 + kb * sfb_step, kSfHi | uint64_t(sfb + kb * 32));
                    if (!narrow) tc_copy_32x128b_x4_pair(sf_cols + 16 + kb * sfb_step + 4, kSfHi | uint64_t(sfb + (4 + kb) * 32));
                    mma_nvfp4_pair(d, da + adv, db + adv, idesc, acc, sf_cols + kb * 4, sf_cols + 16 + kb * sfb_step);
                  }
                }
              }
              tc_commit_pair(smem_u32(&sh->empty[s]), 3);
            }
            if (ks == k_stages - 1) tc_commit_pair(smem_u32(&sh->acc_full[a]), 3);
          }
          // no __syncwarp here: the vote at the top of the next stage (or the accumulator wait) reconverges the warp
          s = s_next;
          ph = ph_next;
        }
      }
    }
  } else if (warp >= 12) {
    reg_dec<kRegsLean>();
    // ------------------------------------------------------------ W4A8 nibbles -> int8 rows of the B tile (both CTAs)
    if constexpr (W4) {
      // q = clamp(rint(codebook[code] * e4m3(scale)), -127, 127) (dequant_weight_kernel, src/cuda/w4a8.cu:44-68) through a
      // table q[scale byte][code] built once per CTA, as in the stand-alone unpacker: a group of 16 weights is one 16-byte
      // table row and byte-permute lookups. Per weight row of the CTA's 128 and stage: 64 bytes of nibbles and 8 scale
      // bytes in, 128 bytes out, written where the 128-byte swizzle puts the row's eight 16-byte units.
      __shared__ __align__(16) uint8_t table[256 * 16];
      const int et = threadIdx.x - 384;  // 0..127
      for (int e = et; e < 256; e += 128) {
        const float sc = e4m3_decode(uint8_t(e));
        uint32_t w[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float4 c = __ldg(reinterpret_cast<const float4*>(g.w4_codebook) + j);
          const float cc[4] = {c.x, c.y, c.z, c.w};
          uint32_t acc = 0;
#pragma unroll
          for (int i = 0; i < 4; ++i) acc |= uint32_t(uint8_t(max(-127, min(127, __float2int_rn(cc[i] * sc))))) << (8 * i);
          w[j] = acc;
        }
        reinterpret_cast<uint4*>(table)[e] = make_uint4(w[0], w[1], w[2], w[3]);
      }
      asm volatile("bar.sync 2, 128;" ::: "memory");
      const uint4* trow = reinterpret_cast<const uint4*>(table);
      const uint32_t b_full_leader = map_to_rank(smem_u32(&sh->sf_full[0]), 0);
      const int groups_per_row = g.K / 16;
      // Warp e of the four takes every fourth stage whole (its lanes walk the 128 rows in four passes of 32), so that four
      // stages are being expanded at a time: a stage's chain -- wait, loads, lookups, stores, the fence for the tensor
      // core's proxy, the arrival -- is several times longer than the 512 cycles the stage's MMAs take, and with one row per
      // thread and all four warps on the same stage the chains ran one after the other.
      const int ew = warp - 12;
      const int my_tiles = pair < num_work ? (num_work - pair + num_pairs - 1) / num_pairs : 0;
      const uint32_t total_iters = uint32_t(my_tiles) * uint32_t(k_stages);
      auto scale_rows = [&](uint32_t it, uint2 (&sc)[4]) {  // the 8 scale bytes of this lane's four rows for pipeline iteration `it`
        const int seq = int(it / uint32_t(k_stages)), ks = int(it - uint32_t(seq) * uint32_t(k_stages));
        int tm, tn, n_off, n_cols;
        work_item(pair + seq * num_pairs, tm, tn, n_off, n_cols);
#pragma unroll
        for (int p4 = 0; p4 < 4; ++p4) {
          const int wrow = min(tn * BN + int(rank) * (BN / 2) + p4 * 32 + lane, g.N - 1);
          sc[p4] = __ldg(reinterpret_cast<const uint2*>(g.w4_gscale + size_t(wrow) * groups_per_row + ks * 8));
        }
      };
      uint2 sc_next[4];
      if (uint32_t(ew) < total_iters) scale_rows(uint32_t(ew), sc_next);
      bool ok = true;
      for (uint32_t it = uint32_t(ew); it < total_iters && ok; it += 4) {
        const int s = it % C::kStages;
        const uint32_t ph = (it / C::kStages) & 1;
        uint2 sc[4];
#pragma unroll
        for (int p4 = 0; p4 < 4; ++p4) sc[p4] = sc_next[p4];
        if (it + 4 < total_iters) scale_rows(it + 4, sc_next);
        // the nibbles have landed; the producer issued them only after empty[s], so the B area is free as well
        if (!(ok = wait_barrier_warp(smem_u32(&sh->w4_full[s]), ph, sh, g.status, 6))) break;
        uint8_t* stage = smem + s * C::kStageBytes;
#pragma unroll
        for (int p4 = 0; p4 < 4; ++p4) {
          const int r = p4 * 32 + lane;
          const uint4* src = reinterpret_cast<const uint4*>(stage + C::kStageA + C::kStageB) + r * 4;  // 64 bytes per row
          uint8_t* dst = stage + C::kStageA + r * kSlabBytes;
          const uint32_t swz = uint32_t(r & 7);
          const uint32_t scw[2] = {sc[p4].x, sc[p4].y};
#pragma unroll
          for (int q4 = 0; q4 < 4; ++q4) {  // 16 bytes of nibbles = two groups of 16 weights
            const uint4 raw = src[q4];
            const uint32_t words[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
            for (int h = 0; h < 2; ++h) {
              const int grp = q4 * 2 + h;
              const uint4 row = trow[(scw[grp >> 2] >> (8 * (grp & 3))) & 0xFFu];
              uint32_t o[4];
#pragma unroll
              for (int w = 0; w < 4; ++w) {
                const uint32_t codes = (words[h * 2 + (w >> 1)] >> (16 * (w & 1))) & 0xFFFFu;  // four nibbles = elements 4w .. 4w+3
                const uint32_t sel = codes & 0x7777u;                                          // index inside an 8-entry half
                const uint32_t lo = __byte_perm(row.x, row.y, sel), hi = __byte_perm(row.z, row.w, sel);
                o[w] = __byte_perm(lo, hi, 0x3210u | ((codes & 0x8888u) >> 1));  // byte i from `hi` when bit 3 of code i is set
              }
              *reinterpret_cast<uint4*>(dst + ((uint32_t(grp) ^ swz) << 4)) = make_uint4(o[0], o[1], o[2], o[3]);
            }
          }
        }
        fence_proxy_async();  // the rows are read by the tensor core's proxy
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(b_full_leader + uint32_t(s) * 8u);
      }
    }
  } else {
    reg_inc<kRegsEpilogue>();
    // ------------------------------------------------------------ epilogue (8 warps, both CTAs)
    const int quad = warp & 3;
    const int half = (warp - 4) >> 2;
    const int et = threadIdx.x - 128;
    uint32_t tile_it = 0;
    bool ok = true;
    const bool vec_ok = (g.N % 8 == 0) && ((reinterpret_cast<uintptr_t>(g.y) & 15) == 0) && (g.ldy % 8 == 0);
    const bool has_bias = g.bias != nullptr;
    const uint32_t acc_empty_leader[2] = {map_to_rank(smem_u32(&sh->acc_empty[0]), 0), map_to_rank(smem_u32(&sh->acc_empty[1]), 0)};
    for (int t = pair; t < num_work && ok; t += num_pairs, ++tile_it) {
      int tm, tn, n_off, n_cols_rt;
      work_item(t, tm, tn, n_off, n_cols_rt);
      const int n_cols = TAIL ? n_cols_rt : BN;  // a compile-time constant without the tail split
      const int col_base = tn * BN + n_off;      // first output column of this work item
      const int a = tile_it % ACC;
      const uint32_t aph = (tile_it / ACC) & 1;
      float* cs_s = sh->col_scale[tile_it & 1];
      float* bs_s = sh->bias[tile_it & 1];
      if (et < n_cols) {
        const int col = swiglu ? (et < BN / 2 ? tn * (BN / 2) + et : inner + tn * (BN / 2) + et - BN / 2) : col_base + et;
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
      if constexpr (EPI == kEpiGated) {
        // Gated residual: the epilogue will read-modify-write this tile of y. Ask L2 for it now, a whole main loop
        // ahead, so those reads do not pay HBM latency on the store path (128 rows x BN bf16 = BN/64 lines per row).
        const int kLinesPerRow = n_cols / 64;
        for (int l = et; l < kBM * kLinesPerRow; l += 256) {
          const int pr = tm * kPairBM + int(rank) * kBM + l / kLinesPerRow, pc = col_base + (l % kLinesPerRow) * 64;
          if (pr < g.M && pc < g.N) asm volatile("prefetch.global.L2 [%0];" ::"l"(g.y + size_t(pr) * g.ldy + pc));
        }
      }
      asm volatile("bar.sync 1, 256;" ::: "memory");
      if (!(ok = wait_barrier(smem_u32(&sh->acc_full[a]), aph, sh, g.status, 4))) break;
      tc_fence_after_sync();
      const int tile_row0 = tm * kPairBM + int(rank) * kBM;
      const int row = tile_row0 + quad * 32 + lane;
      const bool row_ok = row < g.M;
      const float rs = (KIND == kI8 && row_ok) ? __ldg(g.row_scale + row) : 1.0f;
      __nv_bfloat16* yrow = g.y + size_t(row_ok ? row : 0) * g.ldy;
      const int warp_row0 = tile_row0 + quad * 32;
      const int rows_ok = max(0, min(32, g.M - warp_row0));
      __nv_bfloat16* ywarp = g.y + size_t(min(warp_row0, g.M - 1)) * g.ldy;
      uint4* stage_w = reinterpret_cast<uint4*>(smem + C::kStages * C::kStageBytes + C::kBarrierBytes) + (warp - 4) * 128;
      const int kTileChunks = n_cols / 32;
      constexpr int kMaxJ = (BN / 32 + 1) / 2;
      const uint32_t tbase = tmem + a * BN + (uint32_t(quad * 32) << 16);
      int gate_idx[4] = {0, 0, 0, 0};
      const float* gate_row = nullptr;
      if constexpr (EPI == kEpiGated) {
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
      if (lane == 0) mbar_arrive_cluster(acc_empty_leader[a]);
      if constexpr (swiglu) {
        // this warp holds gate chunks half, half + 2 (r[0], r[1]) and their up chunks half + 4, half + 6 (r[2], r[3])
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          const int c = half + 2 * j;
          uint4 pg[4], pu[4], po[4];
          if (has_bias) {
            pack_chunk<KIND, true, false>(r[j], rs, cs_s + c * 32, bs_s + c * 32, pg);
            pack_chunk<KIND, true, false>(r[j + 2], rs, cs_s + (c + 4) * 32, bs_s + (c + 4) * 32, pu);
          } else {
            pack_chunk<KIND, false, false>(r[j], rs, cs_s + c * 32, bs_s + c * 32, pg);
            pack_chunk<KIND, false, false>(r[j + 2], rs, cs_s + (c + 4) * 32, bs_s + (c + 4) * 32, pu);
          }
          swiglu_chunk(pg, pu, po);
          flush_chunk(po, stage_w, ywarp + tn * (BN / 2) + c * 32, size_t(g.ldy), rows_ok, lane);
        }
        continue;
      }
#pragma unroll
      for (int j = 0; j < kMaxJ; ++j) {
        const int c = half + 2 * j;
        const int col0 = col_base + c * 32;
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
          if constexpr (EPI == kEpiGated)
            flush_chunk(packed, stage_w, ywarp + col0, size_t(g.ldy), rows_ok, lane, g.gate + col0, size_t(g.N), gate_idx);
          else
            flush_chunk(packed, stage_w, ywarp + col0, size_t(g.ldy), rows_ok, lane);
        } else if (row_ok) {
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
  cluster_sync_all();  // the pair's MMAs, copies and remote arrivals are all behind both CTAs here
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc_pair(tmem, C::kTmemCols);
  }
}

// Scale array of one operand in the 128x4 tiling, seen as [row tiles][K/64 atoms x 512 bytes] of 8-byte elements;
// a box is `tiles` row tiles x 4 atoms (2 KB each), unswizzled, zero beyond the array.
CUtensorMap make_scale_map(const void* base, size_t row_tiles, size_t k_atoms, int tiles) {
  if (reinterpret_cast<uintptr_t>(base) % 16 != 0) throw std::invalid_argument("sfq gemm: scale arrays must be 16-byte aligned");
  CUtensorMap m;
  const cuuint64_t dims[2] = {k_atoms * 64, row_tiles};
  const cuuint64_t strides[1] = {k_atoms * 512};
  const cuuint32_t box[2] = {256, cuuint32_t(tiles)};
  const cuuint32_t elem[2] = {1, 1};
  const CUresult r = encode_fn()(&m, CU_TENSOR_MAP_DATA_TYPE_UINT64, 2, const_cast<void*>(base), dims, strides, box, elem,
                                 CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                 CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) throw std::runtime_error("sfq gemm: cuTensorMapEncodeTiled failed for a scale array (" + std::to_string(int(r)) + ")");
  return m;
}

template <int KIND, int ACC, int EPI> int max_pairs() {  // the same for both TAIL variants
  // Clusters of two need both CTAs in one GPC; ask the runtime how many pairs fit at once.
  static PerDevice<int> cache;
  return cache.get([] {
    using C = PairCfg<KIND, ACC>;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2 * sm_count());
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = C::kSmemBytes;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = 2;
    attr.val.clusterDim.y = 1;
    attr.val.clusterDim.z = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    int clusters = 0;
    const cudaError_t e = cudaOccupancyMaxActiveClusters(&clusters, gemm_pair_kernel<KIND, ACC, EPI, false>, &cfg);
    if (e != cudaSuccess || clusters <= 0) {
      cudaGetLastError();
      return 0;
    }
    return clusters;
  });
}

template <int KIND, int ACC, int EPI>
bool launch_pair_epi(const void* a, const void* w, size_t row_bytes, const GemmArgs& g, cudaStream_t stream) {
  using C = PairCfg<KIND, ACC>;
  reserve_dynamic_smem(reinterpret_cast<const void*>(&gemm_pair_kernel<KIND, ACC, EPI, false>), C::kSmemBytes, "sfq gemm");
  reserve_dynamic_smem(reinterpret_cast<const void*>(&gemm_pair_kernel<KIND, ACC, EPI, true>), C::kSmemBytes, "sfq gemm");
  const int pairs_fit = max_pairs<KIND, ACC, EPI>();
  if (pairs_fit <= 0) return false;  // no room for clusters of two: the caller uses the one-CTA kernel
  const CUtensorMap ma = make_map(a, size_t(g.M), row_bytes, kBM);
  const CUtensorMap mb = make_map(w, size_t(g.N), row_bytes, kPairBN / 2);
  const CUtensorMap mbn = make_map(w, size_t(g.N), row_bytes, kPairBN / 4);
  CUtensorMap msa = ma, msb = mb, msbn = mb;  // placeholders for the kinds without scales
  if constexpr (KIND == kNvfp4) {
    msa = make_scale_map(g.a_scale_tiled, size_t((g.M + 127) / 128), size_t(g.K / 64), 1);
    msb = make_scale_map(g.w_scale_tiled, size_t(g.N / 128), size_t(g.K / 64), 2);
    msbn = make_scale_map(g.w_scale_tiled, size_t(g.N / 128), size_t(g.K / 64), 1);
  }
  if (g.act == SFQ_ACT_SWIGLU) {
    if (g.N % kPairBN != 0) throw std::invalid_argument("sfq gemm: the SwiGLU epilogue needs N % 256 == 0 (gate and up halves in 128-column blocks)");
    if (g.gate != nullptr) throw std::invalid_argument("sfq gemm: the SwiGLU epilogue cannot be combined with the gated residual");
    if (g.ldy != g.N / 2 || reinterpret_cast<uintptr_t>(g.y) % 16 != 0)
      throw std::invalid_argument("sfq gemm: the SwiGLU epilogue writes [M, N/2], 16-byte aligned");
  }
  const int tiles = ((g.M + kPairBM - 1) / kPairBM) * ((g.N + kPairBN - 1) / kPairBN);  // same count with or without SwiGLU
  int pairs_cap = pairs_fit;
  if (g.max_ctas > 0) pairs_cap = std::max(1, std::min(pairs_cap, g.max_ctas / 2));
  // Tail of the schedule: r tiles are left for the last wave. If they would occupy at most half of the pairs they
  // can be cut in two, so that wave keeps twice as many pairs busy on narrower tiles and ends sooner. That pays
  // while the launch has few waves (the saved third of a wave outweighs the narrow tiles' lower efficiency and the
  // TAIL kernel variant's extra bookkeeping: +3.5 % at 4.3 waves, -1 % at 17.3) and, for nvfp4, only for launches
  // of less than half a wave: a narrow nvfp4 stage is bound by its scale hand-off, not by its MMAs.
  GemmArgs ga = g;
  const int r = tiles % pairs_cap;
  const bool few_waves = KIND == kNvfp4 ? 2 * tiles <= pairs_cap : tiles < 8 * pairs_cap;
  ga.tail_split = g.tail_split >= 0 ? std::min(g.tail_split, tiles) : ((r > 0 && 2 * r <= pairs_cap && few_waves) ? r : 0);
  if (g.act == SFQ_ACT_SWIGLU) ga.tail_split = 0;  // a tile must keep its gate and up halves together
  const int pairs = std::min(tiles + ga.tail_split, pairs_cap);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * pairs);
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = C::kSmemBytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr;
  attr.id = cudaLaunchAttributeClusterDimension;
  attr.val.clusterDim.x = 2;
  attr.val.clusterDim.y = 1;
  attr.val.clusterDim.z = 1;
  cfg.attrs = &attr;
  cfg.numAttrs = 1;
  const cudaError_t e = ga.tail_split > 0
                            ? cudaLaunchKernelEx(&cfg, gemm_pair_kernel<KIND, ACC, EPI, true>, ma, mb, msa, msb, mbn, msbn, ga)
                            : cudaLaunchKernelEx(&cfg, gemm_pair_kernel<KIND, ACC, EPI, false>, ma, mb, msa, msb, mbn, msbn, ga);
  if (e != cudaSuccess) throw std::runtime_error(std::string("sfq gemm: pair launch failed: ") + cudaGetErrorString(e));
  return true;
}

template <int KIND, int ACC>
bool launch_pair(const void* a, const void* w, size_t row_bytes, const GemmArgs& g, cudaStream_t stream) {
  if (g.act == SFQ_ACT_SWIGLU) return launch_pair_epi<KIND, ACC, kEpiSwiglu>(a, w, row_bytes, g, stream);
  if (g.gate != nullptr) return launch_pair_epi<KIND, ACC, kEpiGated>(a, w, row_bytes, g, stream);
  return launch_pair_epi<KIND, ACC, kEpiPlain>(a, w, row_bytes, g, stream);
}

}  // namespace

bool gemm_pair_int8(const int8_t* a, const int8_t* w, const GemmArgs& g, cudaStream_t stream) {
  return launch_pair<kI8, 2>(a, w, size_t(g.K), g, stream);
}
bool gemm_pair_nvfp4(const uint8_t* a, const uint8_t* w, const GemmArgs& g, cudaStream_t stream) {
  return launch_pair<kNvfp4, 1>(a, w, size_t(g.K) / 2, g, stream);
}
bool gemm_pair_bf16(const __nv_bfloat16* a, const __nv_bfloat16* w, const GemmArgs& g, cudaStream_t stream) {
  return launch_pair<kBf16, 2>(a, w, size_t(g.K) * 2, g, stream);
}

bool gemm_pair_w4a8(const int8_t* a, const uint8_t* w_packed, const GemmArgs& g, cudaStream_t stream) {
  using C = PairCfg<kI8, 2, true>;
  if (g.K % kSlabBytes != 0 || g.act == SFQ_ACT_SWIGLU || g.gate != nullptr || !g.w4_gscale || !g.w4_codebook) return false;
  if (reinterpret_cast<uintptr_t>(g.w4_codebook) % 16 != 0 || reinterpret_cast<uintptr_t>(g.w4_gscale) % 8 != 0 ||
      reinterpret_cast<uintptr_t>(w_packed) % 16 != 0)
    throw std::invalid_argument("sfq gemm: W4A8 nibbles and codebook must be 16-byte aligned, the group scales 8-byte aligned");
  auto kernel = gemm_pair_kernel<kI8, 2, kEpiPlain, false, true>;
  reserve_dynamic_smem(reinterpret_cast<const void*>(kernel), C::kSmemBytes, "sfq gemm");
  static PerDevice<int> cache;
  const int pairs_fit = cache.get([&] {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2 * sm_count());
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = C::kSmemBytes;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = 2, attr.val.clusterDim.y = 1, attr.val.clusterDim.z = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    int clusters = 0;
    if (cudaOccupancyMaxActiveClusters(&clusters, kernel, &cfg) != cudaSuccess || clusters <= 0) {
      cudaGetLastError();
      return 0;
    }
    return clusters;
  });
  if (pairs_fit <= 0) return false;
  const CUtensorMap ma = make_map(a, size_t(g.M), size_t(g.K), kBM);
  // nibbles [N, K/2]: boxes of 64 bytes x 128 rows, unswizzled, zero beyond the array
  CUtensorMap mw;
  {
    const cuuint64_t dims[2] = {cuuint64_t(g.K) / 2, cuuint64_t(g.N)};
    const cuuint64_t strides[1] = {cuuint64_t(g.K) / 2};
    const cuuint32_t box[2] = {kSlabBytes / 2, kPairBN / 2};
    const cuuint32_t elem[2] = {1, 1};
    const CUresult r = encode_fn()(&mw, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<uint8_t*>(w_packed), dims, strides, box, elem,
                                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) throw std::runtime_error("sfq gemm: cuTensorMapEncodeTiled failed for the W4A8 nibbles (" + std::to_string(int(r)) + ")");
  }
  const int tiles = ((g.M + kPairBM - 1) / kPairBM) * ((g.N + kPairBN - 1) / kPairBN);
  int pairs_cap = pairs_fit;
  if (g.max_ctas > 0) pairs_cap = std::max(1, std::min(pairs_cap, g.max_ctas / 2));
  GemmArgs ga = g;
  ga.tail_split = 0;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * std::min(tiles, pairs_cap));
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = C::kSmemBytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr;
  attr.id = cudaLaunchAttributeClusterDimension;
  attr.val.clusterDim.x = 2, attr.val.clusterDim.y = 1, attr.val.clusterDim.z = 1;
  cfg.attrs = &attr;
  cfg.numAttrs = 1;
  const cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, ma, mw, ma, ma, ma, ma, ga);
  if (e != cudaSuccess) throw std::runtime_error(std::string("sfq gemm: pair launch failed: ") + cudaGetErrorString(e));
  return true;
}

}  // namespace sfq
