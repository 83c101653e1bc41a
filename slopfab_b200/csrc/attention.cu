// Full (unmasked, non-causal) self-attention with head_dim 128 on tcgen05: out = softmax(q k^T * scale) v per head.
//
// The reference's interface is attention_forward / attention_forward_query_chunk
// (include/slopfab/cuda/attention.cuh:176-196): q, k, v are [seq, heads * 128] row-major bf16, exactly the thirds of the
// fused QKV projection; queries may be a compact chunk of the sequence; no mask exists anywhere in the model.
//
// One CTA owns TWO tiles of 128 queries of one head and walks the keys in tiles of 128 with an online softmax, so that the
// softmax of one query tile runs while the tensor pipe works on the other tile's products:
//   warp 0      TMA producer: both Q tiles once, then a two-stage ring of K tiles [128 keys x 128 d] and V^T tiles
//               [128 d x 128 keys]; V is transposed once per call by transpose_v_kernel so that both products are
//               K-major x K-major, the operand form the GEMM kernels already use
//   warp 1      issues, per key tile j: O0 += P0(j) V(j), S0 = Q0 K(j+1)^T, O1 += P1(j) V(j), S1 = Q1 K(j+1)^T (8 MMAs
//               128x128x16 each). S and O of both query tiles live in TMEM (4 x 128 columns); P is read by the second
//               product straight from TMEM, where it overwrites the first 64 columns of the scores it was computed from
//   warps 4-7   softmax of query tile 0, warps 8-11 of query tile 1 (warps 2-3 only hand their registers over: the
//               softmax warpgroups run with 216 registers, the first warpgroup with 56), one query row per thread with all 128 keys of the
//               tile: S from TMEM, P = exp2(s - m) as bf16 pairs back into TMEM, the running sum, and - only when the
//               tile's probabilities sum to more than 2^15, i.e. the row has outgrown the reference maximum m the
//               accumulator was last scaled to - the true running maximum, a rescale of O in TMEM and the tile's
//               probabilities again. A stale reference changes nothing in exact arithmetic (numerator and denominator
//               carry the same factor); the limit keeps every p far inside the range of bf16 and fp32, and no maximum over
//               the scores is computed on the common path.
// Every wait is bounded; a wait that runs out stores a code in the status word and the CTA leaves.
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cmath>
#include <cstdint>
#include <mutex>
#include <stdexcept>
#include <string>

#include "gemm_common.cuh"
#include "kernels.cuh"
#include "ptx.cuh"
#include "runtime.h"

namespace sfq {
namespace {

using namespace ptx;

constexpr int kTile = 128;             // queries per query tile (two per CTA), keys per step, head_dim
constexpr int kSlab = kTile * 128;     // 128 rows x 128 bytes: 64 bf16 columns of a tile
constexpr int kTileBytes = 2 * kSlab;  // [128 x 128] bf16
constexpr int kAttnThreads = 384;  // warpgroup 0: producer, MMA issuer, two idle warps; warpgroups 1 and 2: the softmax of query tiles 0 and 1
constexpr int kAttnRegsLean = 56, kAttnRegsSoftmax = 216;  // after setmaxnreg: 128 x 56 + 256 x 216 <= 65536
constexpr float kTileSumLimit = 32768.0f;  // a key tile's 128 probabilities may sum to this before the reference maximum moves

struct AttnShared {
  uint64_t q_full, k_full[2], k_empty[2], v_full[2], v_empty[2], s_full[2], p_full[2], pv_done[2];
  uint32_t tmem_base;
  volatile int abort;
};
constexpr int kAttnSmem = 1024 /* alignment slack */ + 6 * kTileBytes /* Q x2, K x2, V^T x2 */ + 1024;

struct AttnArgs {
  __nv_bfloat16* out;
  int ld_out;
  int seq_q, seq_kv;
  int group;         // query heads per key/value head
  float scale_log2;  // scale * log2(e)
  int* status;
};

// `nap` > 0: sleep that many nanoseconds between polls. The softmax warps and the producer wait for long stretches by
// design; polling flat out they would take issue slots from the one warp that feeds the tensor pipe.
template <int nap = 0>
__device__ __forceinline__ bool attn_wait(uint32_t bar, uint32_t parity, AttnShared* sh, int* status, int code) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long start = clock_now();
  for (;;) {
    for (int i = 0; i < 64; ++i) {
      if (mbar_try_wait(bar, parity)) return true;
      if (nap > 0) __nanosleep(nap);
    }
    if (sh->abort) return false;
    if (clock_now() - start > kWaitCycles) {
      atomicCAS(status, 0, code);
      sh->abort = 1;
      return false;
    }
  }
}

__device__ __forceinline__ float max3(float a, float b, float c) {  // one instruction on sm_100
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// 2^x for a pair of arguments on the FMA pipe instead of the special-function unit, which is what the softmax of two
// query tiles saturates (32768 exponentials per key tile at 16 per clock = the 2048 cycles the tile's products take).
// x = n + f with n = round(x), f in [-1/2, 1/2]: a cubic for 2^f (relative error 7.5e-5, a sixtieth of the bf16 rounding
// the result goes through) and n added into the exponent field. Arguments are clamped at -125 below, where the result
// (~2e-38) is as good as the zero the hardware instruction returns, and at 126 above: a row that has outgrown its
// reference by that much must still produce a huge value, which the caller's sum test then catches.
__device__ __forceinline__ f32x2 exp2_pair_fma(f32x2 x) {
  float x0, x1;
  unpack2(x, x0, x1);
  const f32x2 xc = pack2(fminf(fmaxf(x0, -125.0f), 126.0f), fminf(fmaxf(x1, -125.0f), 126.0f));
  const f32x2 magic = pack2(12582912.0f, 12582912.0f);  // 1.5 * 2^23: the sum's low mantissa bits hold round(x)
  const f32x2 t = add2(xc, magic);
  const f32x2 f = sub2(xc, sub2(t, magic));
  f32x2 p = fma2(pack2(0.0551716648f, 0.0551716648f), f, pack2(0.2426111251f, 0.2426111251f));
  p = fma2(p, f, pack2(0.6932609677f, 0.6932609677f));
  p = fma2(p, f, pack2(0.9999280572f, 0.9999280572f));
  float p0, p1, t0, t1;
  unpack2(p, p0, p1);
  unpack2(t, t0, t1);
  return pack2(__int_as_float(__float_as_int(p0) + (__float_as_int(t0) << 23)), __int_as_float(__float_as_int(p1) + (__float_as_int(t1) << 23)));
}
constexpr int kFmaPairsOfFour = 1;  // of every four pairs of probabilities, how many take the FMA-pipe exponential

__global__ void __launch_bounds__(kAttnThreads, 1)
    attention_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                     const __grid_constant__ CUtensorMap map_vt, const AttnArgs g) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* q_s = smem;                    // two query tiles
  uint8_t* k_s = smem + 2 * kTileBytes;   // two stages
  uint8_t* v_s = smem + 4 * kTileBytes;   // two stages
  AttnShared* sh = reinterpret_cast<AttnShared*>(smem + 6 * kTileBytes);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int q0 = blockIdx.x * (2 * kTile);
  const int head = blockIdx.y;
  const int kv_head = head / g.group;
  const int tiles = (g.seq_kv + kTile - 1) / kTile;

  if (threadIdx.x == 0) {
    mbar_init(smem_u32(&sh->q_full), 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(smem_u32(&sh->k_full[i]), 1);
      mbar_init(smem_u32(&sh->k_empty[i]), 1);
      mbar_init(smem_u32(&sh->v_full[i]), 1);
      mbar_init(smem_u32(&sh->v_empty[i]), 1);
      mbar_init(smem_u32(&sh->s_full[i]), 1);   // per query tile: the scores of the current key tile are in TMEM
      mbar_init(smem_u32(&sh->p_full[i]), 4);   // per query tile: its four softmax warps have written P (and rescaled O)
      mbar_init(smem_u32(&sh->pv_done[i]), 1);  // per query tile: O += P V of the current key tile has completed
    }
    sh->abort = 0;
    fence_barrier_init();
    prefetch_tensormap(&map_q);
    prefetch_tensormap(&map_k);
    prefetch_tensormap(&map_vt);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(&sh->tmem_base), 512);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = sh->tmem_base;  // columns: S/P of tile 0 [0,128), of tile 1 [128,256), O of tile 0 [256,384), of tile 1 [384,512)

  // Each role's code sits directly under its warpgroup's setmaxnreg, so the compiler budgets it accordingly.
  if (warp < 4) {
    reg_dec<kAttnRegsLean>();
  if (warp == 0) {
    // ------------------------------------------------------------ producer
    if (lane == 0) {
      mbar_arrive_expect_tx(smem_u32(&sh->q_full), 2 * kTileBytes);
      for (int t = 0; t < 2; ++t) {
        tma_load_2d(smem_u32(q_s + t * kTileBytes), &map_q, head * 256, q0 + t * kTile, smem_u32(&sh->q_full));
        tma_load_2d(smem_u32(q_s + t * kTileBytes + kSlab), &map_q, head * 256 + 128, q0 + t * kTile, smem_u32(&sh->q_full));
      }
      for (int j = 0; j < tiles; ++j) {
        const int st = j & 1;
        const uint32_t ph = ((j >> 1) & 1) ^ 1;
        if (!attn_wait<200>(smem_u32(&sh->k_empty[st]), ph, sh, g.status, 11)) break;
        mbar_arrive_expect_tx(smem_u32(&sh->k_full[st]), kTileBytes);
        tma_load_2d(smem_u32(k_s + st * kTileBytes), &map_k, kv_head * 256, j * kTile, smem_u32(&sh->k_full[st]));
        tma_load_2d(smem_u32(k_s + st * kTileBytes + kSlab), &map_k, kv_head * 256 + 128, j * kTile, smem_u32(&sh->k_full[st]));
        if (!attn_wait<200>(smem_u32(&sh->v_empty[st]), ph, sh, g.status, 12)) break;
        mbar_arrive_expect_tx(smem_u32(&sh->v_full[st]), kTileBytes);
        // V^T: rows are (kv_head, d), columns are keys; 64 keys = 128 bytes per slab
        tma_load_2d(smem_u32(v_s + st * kTileBytes), &map_vt, j * 256, kv_head * kTile, smem_u32(&sh->v_full[st]));
        tma_load_2d(smem_u32(v_s + st * kTileBytes + kSlab), &map_vt, j * 256 + 128, kv_head * kTile, smem_u32(&sh->v_full[st]));
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer (converged warp, one elected lane issues)
    // Issue order per key tile j: O0 += P0(j) V(j); S0 = Q0 K(j+1)^T; O1 += P1(j) V(j); S1 = Q1 K(j+1)^T. The tensor pipe
    // executes what one thread issues in order, so S_t(j+1) overwrites the columns P_t(j) lived in only after the
    // product that read them, and a completed S_t(j+1) also says that O_t holds the sum up to tile j.
    constexpr uint32_t idesc = idesc_bf16(kTile, kTile);
    const uint32_t full_mask = 0xffffffffu;
    // A barrier that has already completed costs one non-suspending probe and a vote; only a real wait takes the polling loop.
    auto wait = [&](uint64_t* bar, uint32_t parity, int code) {
      if (__all_sync(full_mask, mbar_test_wait(smem_u32(bar), parity))) return true;
      return bool(__all_sync(full_mask, attn_wait(smem_u32(bar), parity, sh, g.status, code)));
    };
    bool ok = wait(&sh->q_full, 0, 13);
    auto issue_s = [&](int t, int j) {  // S_t = Q_t K_j^T
      const int st = j & 1;
      // the second query tile reads the K tile the first one has just waited for
      if (t == 0 && !wait(&sh->k_full[st], (j >> 1) & 1, 14)) return false;
      tc_fence_after_sync();
      if (elect_one())  // eight MMAs, the commit for the softmax warps and, behind the second query tile, the one that frees K
        mma_f16_x8_commit(tmem + t * kTile, smem_desc_sw128(smem_u32(q_s + t * kTileBytes)), smem_desc_sw128(smem_u32(k_s + st * kTileBytes)),
                          idesc, 0u, kSlab >> 4, smem_u32(&sh->s_full[t]), smem_u32(&sh->k_empty[st]), t == 1 ? 1u : 0u);
      __syncwarp();
      return true;
    };
    auto issue_pv = [&](int t, int j) {  // O_t += P_t V_j: A = P_t in tensor memory [queries x keys], B = V^T [d x keys]
      const int st = j & 1;
      if (t == 0 && !wait(&sh->v_full[st], (j >> 1) & 1, 16)) return false;
      if (!wait(&sh->p_full[t], j & 1, 17)) return false;
      tc_fence_after_sync();
      if (elect_one())  // 16 keys per MMA: eight 32-bit columns of bf16 pairs
        mma_f16_ts_x8_commit(tmem + 2 * kTile + t * kTile, tmem + t * kTile, smem_desc_sw128(smem_u32(v_s + st * kTileBytes)), idesc,
                             j ? 1u : 0u, kSlab >> 4, smem_u32(&sh->pv_done[t]), smem_u32(&sh->v_empty[st]), t == 1 ? 1u : 0u);
      __syncwarp();
      return true;
    };
    if (ok) ok = issue_s(0, 0) && issue_s(1, 0);
    for (int j = 0; j < tiles && ok; ++j) {
      const bool more = j + 1 < tiles;
      ok = issue_pv(0, j) && (!more || issue_s(0, j + 1)) && issue_pv(1, j) && (!more || issue_s(1, j + 1));
    }
  }
  } else {
    reg_inc<kAttnRegsSoftmax>();
    // ------------------------------------------------------------ softmax, rescale, output
    // Warps 4-7 serve query tile 0, warps 8-11 query tile 1; within a tile a warp owns the 32 rows of the TMEM quadrant
    // it may access (warp index % 4) and a thread one query row with all 128 keys of the tile, so nothing is exchanged
    // between threads. While the softmax of one query tile runs, the tensor pipe works on the other tile's products.
    const int t = (warp - 4) >> 2;
    const int quad = warp & 3;
    const int row = quad * 32 + lane;
    const uint32_t lane_base = uint32_t(quad * 32) << 16;
    const uint32_t tmem_s = tmem + lane_base + t * kTile;
    const uint32_t tmem_o = tmem + lane_base + 2 * kTile + t * kTile;
    float m_used = -INFINITY;  // the maximum the accumulator and the running sum are expressed against (log2 units)
    float l = 0.0f;
    bool ok = true;
    uint32_t r[4][32];
    const f32x2 scale2 = pack2(g.scale_log2, g.scale_log2);
    // p = 2^(s * scale - m) for the 32 keys of chunk c as bf16 pairs, written over columns [16 c, 16 c + 16) of the
    // scores they came from (those columns belong to chunks 0 and 1, which are in registers by then); returns their sum.
    auto emit_chunk = [&](int c, float m, f32x2 sum2) {
      const f32x2 negm2 = pack2(-m, -m);
      uint32_t pk[16];
#pragma unroll
      for (int i = 0; i < 32; i += 2) {
        const f32x2 x = fma2(pack2(__uint_as_float(r[c][i]), __uint_as_float(r[c][i + 1])), scale2, negm2);
        f32x2 p;
        if (((i >> 1) & 3) < kFmaPairsOfFour) {
          p = exp2_pair_fma(x);
        } else {
          float x0, x1;
          unpack2(x, x0, x1);
          p = pack2(fast_exp2(x0), fast_exp2(x1));
        }
        sum2 = add2(sum2, p);
        float p0, p1;
        unpack2(p, p0, p1);
        const __nv_bfloat162 pb = __floats2bfloat162_rn(p0, p1);  // key 2i in the low half: the lower K index
        pk[i >> 1] = *reinterpret_cast<const uint32_t*>(&pb);
      }
      tmem_st_32x16(tmem_s + c * 16, pk);
      return sum2;
    };
    auto mask_chunk = [&](int c, int valid) {  // the keys past the end of the sequence (last tile only)
#pragma unroll
      for (int i = 0; i < 32; ++i)
        if (c * 32 + i >= valid) r[c][i] = __float_as_uint(-INFINITY);
    };
    auto chunk_max = [&](int c) {
      float m4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};  // four short chains instead of one of 32 steps
#pragma unroll
      for (int i = 0; i < 32; i += 8)
#pragma unroll
        for (int k = 0; k < 4; ++k) m4[k] = max3(m4[k], __uint_as_float(r[c][i + 2 * k]), __uint_as_float(r[c][i + 2 * k + 1]));
      return fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3]));
    };
    for (int j = 0; j < tiles; ++j) {
      if (!(ok = __all_sync(0xffffffffu, attn_wait<40>(smem_u32(&sh->s_full[t]), j & 1, sh, g.status, 18)))) break;
      tc_fence_after_sync();
      const int valid = g.seq_kv - j * kTile;  // keys of this tile that exist
      // The probabilities are computed against the reference maximum the accumulator was last scaled to, which is known
      // before the tile arrives: chunk c is exponentiated while chunk c + 1 is still on its way out of tensor memory. No
      // maximum is taken on this path: that the reference is still good enough is read off the tile's sum of probabilities.
      f32x2 sum2 = pack2(0.0f, 0.0f);
      tmem_ld_32x32(tmem_s, r[0]);
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        tmem_ld_wait();
        if (c + 1 < 4) tmem_ld_32x32(tmem_s + (c + 1) * 32, r[c + 1]);
        if (valid < kTile) mask_chunk(c, valid);
        if (j > 0) sum2 = emit_chunk(c, m_used, sum2);
      }
      float sum0, sum1;
      unpack2(sum2, sum0, sum1);
      float tile_sum = sum0 + sum1;
      const bool over = j == 0 || !(tile_sum <= kTileSumLimit);  // the first tile; a row that outgrew its reference; inf or NaN
      if (__any_sync(0xffffffffu, over)) {
        // Rare after the first tiles. The reference becomes the running maximum. S_t(j) was issued behind O_t += P_t V(j-1),
        // so its completion says that O_t is at rest. The warp rescales its 32 rows together (the TMEM accesses are
        // warp-wide; rows within their limit use a factor of 1) and computes the tile's probabilities again against the new
        // reference -- every score is still in registers -- over the ones just written.
        float mx = -INFINITY;
#pragma unroll
        for (int c = 0; c < 4; ++c) mx = fmaxf(mx, chunk_max(c));
        const float m_new = over ? fmaxf(m_used, mx * g.scale_log2) : m_used;  // scale > 0: the maximum commutes with it
        if (j > 0) {
          const float f = over ? fast_exp2(m_used - m_new) : 1.0f;
          l *= f;
          uint32_t o[32];
#pragma unroll 1
          for (int c = 0; c < 4; ++c) {
            tmem_ld_32x32(tmem_o + c * 32, o);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * f);
            tmem_st_32x32(tmem_o + c * 32, o);
          }
        }
        m_used = m_new;
        sum2 = pack2(0.0f, 0.0f);
#pragma unroll
        for (int c = 0; c < 4; ++c) sum2 = emit_chunk(c, m_used, sum2);
        unpack2(sum2, sum0, sum1);
        tile_sum = sum0 + sum1;
      }
      l += tile_sum;
      tmem_st_wait();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&sh->p_full[t]));
    }
    if (ok && (ok = __all_sync(0xffffffffu, attn_wait(smem_u32(&sh->pv_done[t]), (tiles - 1) & 1, sh, g.status, 20)))) {
      tc_fence_after_sync();
      const float inv = 1.0f / l;
      const int qrow = q0 + t * kTile + row;
      const bool row_ok = qrow < g.seq_q;
      __nv_bfloat16* dst = g.out + size_t(row_ok ? qrow : 0) * g.ld_out + head * kTile;
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint32_t o[32];
        tmem_ld_32x32(tmem_o + c * 32, o);
        tmem_ld_wait();
        if (row_ok) {
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            uint32_t w[4];
#pragma unroll
            for (int h = 0; h < 4; ++h) {
              const __nv_bfloat162 v = __floats2bfloat162_rn(__uint_as_float(o[q * 8 + 2 * h]) * inv, __uint_as_float(o[q * 8 + 2 * h + 1]) * inv);
              w[h] = *reinterpret_cast<const uint32_t*>(&v);
            }
            *reinterpret_cast<uint4*>(dst + c * 32 + q * 8) = make_uint4(w[0], w[1], w[2], w[3]);
          }
        }
      }
      tc_fence_before_sync();
    }
  }
  if (sh->abort) {
    // Leaving early: loads may still be in flight into this CTA's shared memory; give them far more time than a
    // load takes before the memory is released.
    const long long start = clock_now();
    while (clock_now() - start < 4000000ll) {
    }
  }
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem, 512);
  }
}

// V [seq, width] (row pitch ld_v) -> V^T [width, ld_t] with the columns [seq, ld_t) zeroed.
__global__ void __launch_bounds__(256) transpose_v_kernel(const __nv_bfloat16* __restrict__ v, int ld_v, __nv_bfloat16* __restrict__ vt, int ld_t,
                                                          int seq, int width) {
  __shared__ __nv_bfloat16 tile[64][66];
  const int s0 = blockIdx.x * 64, w0 = blockIdx.y * 64;
  for (int i = threadIdx.x; i < 64 * 64; i += 256) {
    const int rs = i >> 6, cw = i & 63;
    tile[rs][cw] = (s0 + rs < seq && w0 + cw < width) ? v[size_t(s0 + rs) * ld_v + w0 + cw] : __float2bfloat16(0.0f);
  }
  __syncthreads();
  for (int i = threadIdx.x; i < 64 * 64; i += 256) {
    const int rw = i >> 6, cs = i & 63;
    if (w0 + rw < width && s0 + cs < ld_t) vt[size_t(w0 + rw) * ld_t + s0 + cs] = tile[cs][rw];
  }
}

// [rows, cols] bf16 with a row pitch, boxes of {64 columns, 128 rows}, 128-byte swizzle, zero fill outside.
CUtensorMap make_attn_map(const void* base, size_t rows, size_t cols, size_t pitch_elems) {
  if (reinterpret_cast<uintptr_t>(base) % 16 != 0 || (pitch_elems * 2) % 16 != 0)
    throw std::invalid_argument("sfq attention: operand base and row pitch must be 16-byte aligned for TMA");
  CUtensorMap m;
  const cuuint64_t dims[2] = {cols * 2, rows};
  const cuuint64_t strides[1] = {pitch_elems * 2};
  const cuuint32_t box[2] = {128, cuuint32_t(kTile)};
  const cuuint32_t elem[2] = {1, 1};
  const CUresult r = encode_fn()(&m, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, elem,
                                 CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                 CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) throw std::runtime_error("sfq attention: cuTensorMapEncodeTiled failed (" + std::to_string(int(r)) + ")");
  return m;
}

size_t align256(size_t n) { return (n + 255) / 256 * 256; }
int padded_keys(int seq_kv) { return (seq_kv + 63) / 64 * 64; }

}  // namespace

size_t attention_workspace_bytes(int seq_kv, int kv_heads, int head_dim) {
  if (seq_kv <= 0 || kv_heads <= 0 || head_dim != kTile) throw std::invalid_argument("sfq attention: head_dim must be 128 and the extents positive");
  return align256(size_t(kv_heads) * kTile * padded_keys(seq_kv) * sizeof(__nv_bfloat16));
}

void attention_forward(const __nv_bfloat16* q, int ld_q, const __nv_bfloat16* k, const __nv_bfloat16* v, int ld_kv, __nv_bfloat16* out, int ld_out,
                       int seq_q, int seq_kv, int heads, int kv_heads, int head_dim, float scale, void* workspace, size_t workspace_bytes,
                       cudaStream_t stream) {
  if (seq_q <= 0) return;
  if (head_dim != kTile) throw std::invalid_argument("sfq attention: only head_dim 128 is built");
  if (seq_kv <= 0 || heads <= 0 || kv_heads <= 0 || heads % kv_heads != 0) throw std::invalid_argument("sfq attention: bad extents");
  if (!q || !k || !v || !out || !workspace) throw std::invalid_argument("sfq attention: null operand");
  if (ld_q < heads * kTile || ld_kv < kv_heads * kTile || ld_out < heads * kTile || ld_out % 8 != 0 || reinterpret_cast<uintptr_t>(out) % 16 != 0)
    throw std::invalid_argument("sfq attention: row pitches must cover heads * 128 columns and keep 16-byte alignment");
  if (workspace_bytes < attention_workspace_bytes(seq_kv, kv_heads, head_dim)) throw std::invalid_argument("sfq attention: workspace too small");
  if (out == q || out == k || out == v) throw std::invalid_argument("sfq attention: out may not alias q, k or v");
  if ((seq_q + kTile - 1) / kTile > 0x7FFFFFFF / 2 || heads > 65535) throw std::invalid_argument("sfq attention: too many query tiles or heads");
  reserve_dynamic_smem(reinterpret_cast<const void*>(&attention_kernel), kAttnSmem, "sfq attention");

  const int ld_t = padded_keys(seq_kv);
  __nv_bfloat16* vt = static_cast<__nv_bfloat16*>(workspace);
  const int width = kv_heads * kTile;
  transpose_v_kernel<<<dim3((ld_t + 63) / 64, (width + 63) / 64), 256, 0, stream>>>(v, ld_kv, vt, ld_t, seq_kv, width);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) throw std::runtime_error(std::string("sfq attention: launch failed: ") + cudaGetErrorString(e));

  const CUtensorMap mq = make_attn_map(q, size_t(seq_q), size_t(heads) * kTile, size_t(ld_q));
  const CUtensorMap mk = make_attn_map(k, size_t(seq_kv), size_t(kv_heads) * kTile, size_t(ld_kv));
  const CUtensorMap mv = make_attn_map(vt, size_t(width), size_t(ld_t), size_t(ld_t));
  AttnArgs a;
  a.out = out, a.ld_out = ld_out, a.seq_q = seq_q, a.seq_kv = seq_kv, a.group = heads / kv_heads;
  a.scale_log2 = (scale > 0.0f ? scale : 1.0f / sqrtf(float(head_dim))) * 1.4426950408889634f;
  a.status = device_status_word();
  attention_kernel<<<dim3((seq_q + 2 * kTile - 1) / (2 * kTile), heads), kAttnThreads, kAttnSmem, stream>>>(mq, mk, mv, a);
  e = cudaGetLastError();
  if (e != cudaSuccess) throw std::runtime_error(std::string("sfq attention: launch failed: ") + cudaGetErrorString(e));
}

}  // namespace sfq
