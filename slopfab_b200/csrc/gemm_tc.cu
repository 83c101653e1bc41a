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
// a commit releases each stage back to the producer. Warps 2-9 drain a finished
// accumulator with tcgen05.ld, apply the fused epilogue and store bf16, while
// the MMA warp already fills the other accumulator buffer.
//
// Every wait is bounded: a barrier that does not complete within kWaitCycles
// makes the waiting thread record a code in the status word, raise the CTA's
// abort flag and fall through to the common exit, where the producer waits
// (bounded) for its own copies in flight and TMEM is released.
#include "gemm_tc.cuh"

#include <cuda_bf16.h>

#include <mutex>
#include <stdexcept>
#include <string>

#include "ptx.cuh"

namespace sfq {
namespace {

using namespace ptx;

constexpr int kBM = 128;             // rows of a tile = TMEM lanes
constexpr int kSlabBytes = 128;      // bytes of K per row per stage (one swizzle atom)
constexpr int kMmaKBytes = 32;       // bytes of K one tcgen05.mma consumes, every kind
constexpr int kThreads = 384;        // producer warp, MMA warp, eight epilogue warps, two scale-copy warps (nvfp4)
constexpr long long kWaitCycles = 2000000000ll;  // ~1 s: far above any legitimate wait

enum Kind { kI8 = 0, kNvfp4 = 1, kBf16 = 2 };

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
  static constexpr int kSfSlots = 4;  // scale slots in flight: copies of stage it+3 may run while stage it multiplies
  static_assert(kAccCols + kSfSlots * kSfSlotCols <= 512, "TMEM budget");
  static_assert(kStages >= 2, "pipeline needs at least two stages");
};

struct Shared {  // lives after the stage ring
  uint64_t full[8];
  uint64_t empty[8];
  uint64_t acc_full[2];
  uint64_t acc_empty[2];
  uint64_t sf_full[4];   // nvfp4: scale factors of a stage are in TMEM slot (stage % 4)
  uint64_t sf_empty[4];  // nvfp4: the MMAs that read that slot have completed
  uint32_t tmem_base;
  volatile int abort;
  alignas(16) float col_scale[2][256];  // per-column epilogue operands of the tile being drained
  alignas(16) float bias[2][256];
};

// Bounded wait. Returns false when the CTA is aborting.
__device__ __forceinline__ bool wait_barrier(uint32_t bar, uint32_t parity, Shared* sh, int* status, int code) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long start = clock_now();
  for (;;) {
    for (int i = 0; i < 64; ++i)
      if (mbar_try_wait(bar, parity)) return true;
    if (sh->abort) return false;
    if (clock_now() - start > kWaitCycles) {
      atomicCAS(status, 0, code);
      sh->abort = 1;
      return false;
    }
  }
}

__device__ __forceinline__ float gelu_tanh_ref(float v) {
  // 0.5 v (1 + tanh(k (v + 0.044715 v^3))), evaluated in the association order of
  // gelu_tanh_kernel (src/cuda/nn_pointwise.cu:74-81) so the bits agree.
  constexpr float k = 0.7978845608028654f;
  return 0.5f * v * (1.0f + tanhf(k * (v + 0.044715f * v * v * v)));
}

// Rounding points of the epilogue, as in the reference: the GEMM result is rounded to bf16 (output_bf16 /
// the GEMM's own store), the bias is added to that bf16 value and re-rounded (add_bias_kernel,
// src/cuda/linear_weights.cu:483-491), and GELU runs in place on the bf16 result.

// Epilogue arithmetic for 32 consecutive columns of one row (a thread owns a ROW in TMEM): scale, round to
// bf16, [add bias, re-round], [GELU, re-round]; the result stays in registers as four 16-byte units.
// `cs`/`bs` point at this chunk's column operands in shared memory (broadcast reads). The rounding points
// are those of `finish`.
template <int KIND, bool BIAS, bool GELU>
__device__ __forceinline__ void pack_chunk(const uint32_t (&r)[32], float rs, const float* cs, const float* bs,
                                           uint4 (&out)[4]) {
#pragma unroll
  for (int v = 0; v < 4; ++v) {
    const float4 c0 = *reinterpret_cast<const float4*>(cs + v * 8), c1 = *reinterpret_cast<const float4*>(cs + v * 8 + 4);
    const float c[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
    float b[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    if constexpr (BIAS) {
      const float4 b0 = *reinterpret_cast<const float4*>(bs + v * 8), b1 = *reinterpret_cast<const float4*>(bs + v * 8 + 4);
      b[0] = b0.x, b[1] = b0.y, b[2] = b0.z, b[3] = b0.w, b[4] = b1.x, b[5] = b1.y, b[6] = b1.z, b[7] = b1.w;
    }
    __nv_bfloat162* pp = reinterpret_cast<__nv_bfloat162*>(&out[v]);
#pragma unroll
    for (int h = 0; h < 4; ++h) {
      float lo, hi;
      if constexpr (KIND == kI8) {
        lo = (float(int32_t(r[v * 8 + 2 * h])) * rs) * c[2 * h];
        hi = (float(int32_t(r[v * 8 + 2 * h + 1])) * rs) * c[2 * h + 1];
      } else if constexpr (KIND == kNvfp4) {
        lo = __uint_as_float(r[v * 8 + 2 * h]) * c[2 * h];
        hi = __uint_as_float(r[v * 8 + 2 * h + 1]) * c[2 * h + 1];
      } else {
        lo = __uint_as_float(r[v * 8 + 2 * h]);
        hi = __uint_as_float(r[v * 8 + 2 * h + 1]);
      }
      __nv_bfloat162 o = __floats2bfloat162_rn(lo, hi);  // the GEMM's own bf16 store
      if constexpr (BIAS) {
        const float2 f = __bfloat1622float2(o);
        o = __floats2bfloat162_rn(f.x + b[2 * h], f.y + b[2 * h + 1]);  // add_bias re-rounds
      }
      if constexpr (GELU) {
        const float2 f = __bfloat1622float2(o);
        o = __floats2bfloat162_rn(gelu_tanh_ref(f.x), gelu_tanh_ref(f.y));
      }
      pp[h] = o;
    }
  }
}

// Writes one warp's 32 rows x 32 bf16 columns. Storing straight from registers would scatter every store
// instruction over 32 rows, so the block goes through a 2 KB shared-memory transpose (16-byte units
// XOR-swizzled with the row, both phases bank-conflict free) and each instruction then writes 64 contiguous
// bytes of 8 rows. `dst` = global address of (first row of the warp, first column of the chunk).
__device__ __forceinline__ void flush_chunk(const uint4 (&packed)[4], uint4* stage, __nv_bfloat16* dst, size_t ldy,
                                            int rows_ok, int lane) {
#pragma unroll
  for (int v = 0; v < 4; ++v) stage[lane * 4 + (v ^ ((lane >> 1) & 3))] = packed[v];
  __syncwarp();
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int row = 8 * i + (lane >> 2), unit = lane & 3;
    const uint4 val = stage[row * 4 + (unit ^ ((row >> 1) & 3))];
    if (row < rows_ok) *reinterpret_cast<uint4*>(dst + size_t(row) * ldy + unit * 8) = val;
  }
  __syncwarp();  // the block is reused by the next chunk
}

template <int KIND, int BN, int ACC>
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
    for (int i = 0; i < 4; ++i) {
      mbar_init(smem_u32(&sh->sf_full[i]), 2);
      mbar_init(smem_u32(&sh->sf_empty[i]), 1);
    }
    sh->abort = 0;
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

  if (warp == 0 && lane == 0) {
    // ------------------------------------------------------------ producer
    uint32_t it = 0;  // running stage counter
    bool ok = true;
    for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
      int tm, tn;
      tile_coords(t, tm, tn);
      for (int ks = 0; ks < k_stages; ++ks, ++it) {
        const int s = it % C::kStages;  // kStages is a compile-time constant
        const uint32_t ph = (it / C::kStages) & 1;
        if (!(ok = wait_barrier(smem_u32(&sh->empty[s]), ph ^ 1, sh, g.status, 1))) break;
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
        tma_load_2d(smem_u32(stage), &map_a, ks * kSlabBytes, tm * kBM, bar);
        tma_load_2d(smem_u32(stage + C::kStageA), &map_b, ks * kSlabBytes, tn * BN, bar);
        if constexpr (KIND == kNvfp4) {
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
    }
    if (!ok) {
      // Aborting: let copies already in flight land before the CTA's shared memory is released.
      const long long start = clock_now();
      for (uint32_t back = 1; back <= uint32_t(C::kStages) && back <= it; ++back) {
        const uint32_t j = it - back;
        const uint32_t bar = smem_u32(&sh->full[j % C::kStages]);
        while (!mbar_try_wait(bar, (j / C::kStages) & 1) && clock_now() - start < kWaitCycles / 4) {
        }
      }
    }
  } else if (warp == 1 && lane == 0) {
    // ------------------------------------------------------------ MMA issuer
    constexpr uint32_t idesc = KIND == kI8 ? idesc_i8(kBM, BN) : (KIND == kNvfp4 ? idesc_nvfp4(kBM, BN) : idesc_bf16(kBM, BN));
    // The issuing thread is a single lane: every instruction between two MMAs is serial latency on the
    // tensor pipe's critical path. So: running counters instead of divisions, descriptor low words derived
    // by one add per stage, and a fully unrolled four-MMA body for full stages.
    bool ok = true;
    const uint32_t a_base = smem_u32(smem) >> 4;                       // start-address fields, 16-byte units
    const uint32_t b_base = smem_u32(smem + C::kStageA) >> 4;
    constexpr uint32_t kStageStep = C::kStageBytes >> 4;
    constexpr uint64_t kDescHi = (uint64_t(1024 >> 4) << 32) | (uint64_t(1) << 46) | (uint64_t(2) << 61);
    const int last_valid = min(4, (row_bytes - (k_stages - 1) * kSlabBytes + kMmaKBytes - 1) / kMmaKBytes);
    int s = 0;
    uint32_t ph = 0, it = 0, tile_it = 0;
    for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x, ++tile_it) {
      const int a = tile_it % ACC;
      if (!(ok = wait_barrier(smem_u32(&sh->acc_empty[a]), ((tile_it / ACC) & 1) ^ 1, sh, g.status, 2))) break;
      tc_fence_after_sync();
      const uint32_t d = tmem + a * BN;
      for (int ks = 0; ks < k_stages; ++ks, ++it) {
        if (!(ok = wait_barrier(smem_u32(&sh->full[s]), ph, sh, g.status, 3))) break;
        tc_fence_after_sync();
        const uint64_t da = kDescHi | uint64_t(a_base + s * kStageStep);
        const uint64_t db = kDescHi | uint64_t(b_base + s * kStageStep);
        const int kb_valid = ks == k_stages - 1 ? last_valid : 4;
        uint32_t sf_cols = 0;
        if constexpr (KIND == kNvfp4) {
          // The scale-copy warps filled TMEM slot (it & 1) for this stage. A single lane issues one tcgen05
          // instruction every ~45 cycles, so the 12 copies of a stage cannot share a thread with its 4 MMAs.
          sf_cols = tmem + C::kAccCols + (it & 3) * C::kSfSlotCols;
          if (!(ok = wait_barrier(smem_u32(&sh->sf_full[it & 3]), (it >> 2) & 1, sh, g.status, 5))) break;
          tc_fence_after_sync();
        }
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
        tc_commit(smem_u32(&sh->empty[s]));  // stage is free once these MMAs have read it
        if constexpr (KIND == kNvfp4) tc_commit(smem_u32(&sh->sf_empty[it & 3]));
        if (++s == C::kStages) s = 0, ph ^= 1;
      }
      if (ok) tc_commit(smem_u32(&sh->acc_full[a]));
    }
  } else if (warp >= 10) {
    // ------------------------------------------------------------ scale-factor copies (nvfp4 only)
    // Warp 10 handles k-blocks 0,1 of every stage, warp 11 k-blocks 2,3: shared memory -> TMEM with one
    // 32x128b copy per (128-row tile, k-block), then a commit that arrives on sf_full when they have landed.
    if constexpr (KIND == kNvfp4) {
      if (lane == 0) {
        const int part = warp - 10;
        constexpr uint64_t kSfHi = (uint64_t(128 >> 4) << 32) | (uint64_t(1) << 46);
        constexpr uint32_t kStageStep = C::kStageBytes >> 4;
        const uint32_t sfa0 = (smem_u32(smem) + C::kStageA + C::kStageB) >> 4;
        const int last_valid = min(4, (row_bytes - (k_stages - 1) * kSlabBytes + kMmaKBytes - 1) / kMmaKBytes);
        int s = 0;
        uint32_t ph = 0, it = 0;
        bool ok = true;
        for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
          for (int ks = 0; ks < k_stages; ++ks, ++it) {
            if (!(ok = wait_barrier(smem_u32(&sh->full[s]), ph, sh, g.status, 6))) break;
            if (!(ok = wait_barrier(smem_u32(&sh->sf_empty[it & 3]), ((it >> 2) & 1) ^ 1, sh, g.status, 7))) break;
            tc_fence_after_sync();
            const int kb_valid = ks == k_stages - 1 ? last_valid : 4;
            const uint32_t sf_cols = tmem + C::kAccCols + (it & 3) * C::kSfSlotCols;
            const uint32_t sfa = sfa0 + s * kStageStep;
            const uint32_t sfb = sfa + (C::kStageSfa >> 4);
#pragma unroll
            for (int j = 0; j < 2; ++j) {
              const int kb = part * 2 + j;
              if (kb < kb_valid) {
                tc_copy_32x128b_x4(sf_cols + kb * 4, kSfHi | uint64_t(sfa + kb * 32));
#pragma unroll
                for (int rt = 0; rt < BN / 128; ++rt)
                  tc_copy_32x128b_x4(sf_cols + 16 + kb * (BN / 32) + rt * 4, kSfHi | uint64_t(sfb + (rt * 4 + kb) * 32));
              }
            }
            tc_commit(smem_u32(&sh->sf_full[it & 3]));
            if (++s == C::kStages) s = 0, ph ^= 1;
          }
        }
      }
    }
  } else if (warp >= 2) {
    // ------------------------------------------------------------ epilogue (8 warps)
    // Warp w may only read TMEM lanes [32*(w%4), +32). Two warps share each lane quadrant and take alternate
    // 32-column chunks, so every scheduler holds two epilogue warps and their latencies overlap.
    const int quad = warp & 3;
    const int half = (warp - 2) >> 2;
    const int et = threadIdx.x - 64;  // 0..255 among the epilogue threads
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
      uint4* stage_w = reinterpret_cast<uint4*>(smem + C::kStages * C::kStageBytes + C::kBarrierBytes) + (warp - 2) * 128;
      // This warp takes the 32-column chunks half, half+2, ... of the tile. Phase 1 drains them from TMEM and
      // does the arithmetic, keeping packed bf16 in registers; the accumulator is then handed back to the MMA
      // warp BEFORE phase 2 writes to global memory, so stores never sit on the tensor pipe's critical path.
      constexpr int kTileChunks = BN / 32;
      constexpr int kMaxJ = (kTileChunks + 1) / 2;
      const uint32_t tbase = tmem + a * BN + (uint32_t(quad * 32) << 16);
      uint32_t r[2][32];
      uint4 packed[kMaxJ][4];
      if (half < kTileChunks) tmem_ld_32x32(tbase + half * 32, r[0]);
#pragma unroll
      for (int j = 0; j < kMaxJ; ++j) {
        const int c = half + 2 * j;
        if (c < kTileChunks) {
          tmem_ld_wait();
          if (j + 1 < kMaxJ && c + 2 < kTileChunks) tmem_ld_32x32(tbase + (c + 2) * 32, r[(j + 1) & 1]);  // overlaps the math
          const int lc0 = c * 32;
          if (!has_bias && g.act == SFQ_ACT_NONE)
            pack_chunk<KIND, false, false>(r[j & 1], rs, cs_s + lc0, bs_s + lc0, packed[j]);
          else if (g.act == SFQ_ACT_NONE)
            pack_chunk<KIND, true, false>(r[j & 1], rs, cs_s + lc0, bs_s + lc0, packed[j]);
          else
            pack_chunk<KIND, true, true>(r[j & 1], rs, cs_s + lc0, bs_s + lc0, packed[j]);
        }
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&sh->acc_empty[a]));
#pragma unroll
      for (int j = 0; j < kMaxJ; ++j) {
        const int c = half + 2 * j;
        const int col0 = tn * BN + c * 32;
        if (c >= kTileChunks || col0 >= g.N) continue;  // warp-uniform
        if (vec_ok && col0 + 32 <= g.N) {
          flush_chunk(packed[j], stage_w, ywarp + col0, size_t(g.ldy), rows_ok, lane);
        } else if (row_ok) {  // ragged N or unaligned output: element stores from this thread's own row
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            const uint32_t w4[4] = {packed[j][v].x, packed[j][v].y, packed[j][v].z, packed[j][v].w};
#pragma unroll
            for (int q = 0; q < 8; ++q) {
              const int col = col0 + v * 8 + q;
              if (col < g.N) yrow[col] = __ushort_as_bfloat16((unsigned short)((w4[q >> 1] >> (16 * (q & 1))) & 0xFFFFu));
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

// ------------------------------------------------------------------ host side

using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                              const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                              CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeFn encode_fn() {
  static EncodeFn fn = [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    const cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q);
    if (e != cudaSuccess || q != cudaDriverEntryPointSuccess || p == nullptr)
      throw std::runtime_error("sfq: cuTensorMapEncodeTiled is not available from this driver");
    return reinterpret_cast<EncodeFn>(p);
  }();
  return fn;
}

// A [rows, row_bytes] byte matrix, boxes of {128 bytes, box_rows}, 128-byte swizzle, zero fill outside.
CUtensorMap make_map(const void* base, size_t rows, size_t row_bytes, int box_rows) {
  if (reinterpret_cast<uintptr_t>(base) % 16 != 0 || row_bytes % 16 != 0)
    throw std::invalid_argument("sfq gemm: operand base and row pitch must be 16-byte aligned for TMA");
  CUtensorMap m;
  const cuuint64_t dims[2] = {row_bytes, rows};
  const cuuint64_t strides[1] = {row_bytes};
  const cuuint32_t box[2] = {kSlabBytes, cuuint32_t(box_rows)};
  const cuuint32_t elem[2] = {1, 1};
  const CUresult r = encode_fn()(&m, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, elem,
                                 CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                 CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) throw std::runtime_error("sfq gemm: cuTensorMapEncodeTiled failed (" + std::to_string(int(r)) + ")");
  return m;
}

int sm_count() {
  static int n = [] {
    int dev = 0, v = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev);
    return v > 0 ? v : 148;
  }();
  return n;
}

template <int KIND, int BN, int ACC>
void launch(const void* a, const void* w, size_t row_bytes, const GemmArgs& g, cudaStream_t stream) {
  using C = Cfg<KIND, BN, ACC>;
  static std::once_flag once;
  static cudaError_t attr_err = cudaSuccess;
  std::call_once(once, [] {
    attr_err = cudaFuncSetAttribute(gemm_kernel<KIND, BN, ACC>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes);
  });
  if (attr_err != cudaSuccess) throw std::runtime_error(std::string("sfq gemm: cannot reserve shared memory: ") + cudaGetErrorString(attr_err));
  const CUtensorMap ma = make_map(a, size_t(g.M), row_bytes, kBM);
  const CUtensorMap mb = make_map(w, size_t(g.N), row_bytes, BN);
  const int tiles = ((g.M + kBM - 1) / kBM) * ((g.N + BN - 1) / BN);
  const int grid = g.max_ctas > 0 ? std::min(tiles, g.max_ctas) : std::min(tiles, sm_count());
  gemm_kernel<KIND, BN, ACC><<<grid, kThreads, C::kSmemBytes, stream>>>(ma, mb, g);
  const cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) throw std::runtime_error(std::string("sfq gemm: launch failed: ") + cudaGetErrorString(e));
}

}  // namespace

void gemm_int8(const int8_t* a, const int8_t* w, const GemmArgs& g, cudaStream_t stream) {
  if (g.M <= 0 || g.N <= 0) return;
  if (g.K <= 0 || g.K % 16 != 0) throw std::invalid_argument("sfq gemm int8: K must be a positive multiple of 16");
  if (!a || !w || !g.row_scale || !g.col_scale || !g.y || !g.status)
    throw std::invalid_argument("sfq gemm int8: null operand");
  // 256-wide tiles measured fastest at every DiT shape, small M included (192- and 160-wide tiles fill the
  // last wave better but feed the tensor pipe worse); 128 stays selectable for experiments.
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
  // A 256-wide tile has one accumulator (256 columns + the scale slots); 128-wide tiles have two but feed the
  // tensor pipe less efficiently and measured slower at every DiT shape.
  if (g.tile_n == 128)
    launch<kNvfp4, 128, 2>(a, w, size_t(g.K) / 2, g, stream);
  else
    launch<kNvfp4, 256, 1>(a, w, size_t(g.K) / 2, g, stream);
}

void gemm_bf16(const __nv_bfloat16* a, const __nv_bfloat16* w, const GemmArgs& g, cudaStream_t stream) {
  if (g.M <= 0 || g.N <= 0) return;
  if (g.K <= 0 || g.K % 8 != 0) throw std::invalid_argument("sfq gemm bf16: K must be a positive multiple of 8");
  if (!a || !w || !g.y || !g.status) throw std::invalid_argument("sfq gemm bf16: null operand");
  if (g.tile_n == 128)
    launch<kBf16, 128, 2>(a, w, size_t(g.K) * 2, g, stream);
  else
    launch<kBf16, 256, 2>(a, w, size_t(g.K) * 2, g, stream);
}

}  // namespace sfq
