// Flash-style attention for sm_100a with tcgen05 tensor cores, head dim 64 / 128.
//
// Forward: one CTA per (128-query block, batch*head).  Warps 0-3 own one query row
// per thread (TMEM lane = row, so row max / row sum need no shuffles); warp 4's
// lane 0 issues TMA loads and tcgen05.mma.  Per 128-key block: S = Q K^T into TMEM,
// softmax in registers, P (bf16) staged in shared memory in the 128-byte-swizzled
// K-major layout, PV = P V into TMEM, folded into a register accumulator with the
// running-max rescale.  K is double-buffered, V single-buffered.
//
// Backward: one CTA per (128-key block, batch*head) looping over query blocks;
// five MMAs per step (S, dP, dV += P^T dO, dK += dS^T Q, dQ = dS K).  P and dS are
// written once to shared memory and read both as K-major (dQ) and MN-major
// (dV, dK) operands; dV / dK accumulate in TMEM across the loop, dQ tiles are
// added to an fp32 buffer with vector red.global.add and converted at the end.
//
// Q, K, V are read in place from a packed [B, S, 3*C] projection output through 4-D
// tensor maps, so no head split / transpose copies exist.  All waits are bounded.
// The reference has no attention layer; these kernels serve the transformer
// configurations of the benchmark.
#include "ptx.cuh"
#include "nkb_api.h"

namespace nkb {

constexpr int ATT_THREADS = 160;
constexpr float LOG2E = 1.4426950408889634f;

struct AttnFwdArgs {
  __nv_bfloat16* o;
  float* lse;
  int B, H, S;
  long long ob, oh, os;
  float scale, scale_log2;
  int causal;
  int* status;
};

__device__ __forceinline__ void att_error(int* status, volatile int* abort_flag, int code) {
  *abort_flag = 1;
  if (status) atomicCAS(status, 0, code);
}

// byte offset of 16-byte chunk `chunk` (0..7) of row `r` inside a [rows x 64 bf16]
// 128B-swizzled tile
__device__ __forceinline__ uint32_t sw128_off(int r, int chunk) {
  return uint32_t(r) * 128u + (uint32_t(chunk ^ (r & 7)) << 4);
}

// EXPM selects how probabilities are computed: 0 = fp32 exp2 (one MUFU op per element,
// row sums in registers), 1 = packed half exp2 (two per MUFU op) converted to bf16,
// 2 = packed bf16 exp2.  In modes 1 and 2 the row sums come from an extra MMA of P
// against a tile of ones (16 accumulator columns, one used).  The kernel is bound by the
// exponential unit (128 x 128 exps per key block vs 512 tensor-core cycles), which is
// why halving the MUFU work matters.
template <int D, int EXPM>
__global__ void __launch_bounds__(ATT_THREADS, (D == 64 ? 2 : 1))
attn_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                const __grid_constant__ CUtensorMap tmV, const AttnFwdArgs a) {
  constexpr int TILE = 128 * D * 2;          // bytes of a 128 x D bf16 tile
  constexpr int NKD = D / 64;                // 64-wide sub-tiles along the head dim
  constexpr uint32_t TMEM_COLS = (D == 64) ? 256 : 512;
  constexpr uint32_t O_COL = 128;
  constexpr uint32_t L_COL = 128 + D;  // row sums (modes 1, 2)
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                              ~uintptr_t(1023));
  uint8_t* sQ = smem;
  uint8_t* sK = sQ + TILE;       // two stages
  uint8_t* sV = sK + 2 * TILE;   // one stage
  uint8_t* sP = sV + TILE;       // 128 x 128 bf16
  uint8_t* sOnes = sP + 32768;   // 16 x 128 bf16 ones (K-major B operand of the row-sum MMA)
  uint64_t* bars = reinterpret_cast<uint64_t*>(sOnes + 4096);
  uint64_t* q_full = bars + 0;
  uint64_t* k_full = bars + 1;  // [2]
  uint64_t* v_full = bars + 3;
  uint64_t* s_full = bars + 4;
  uint64_t* p_full = bars + 5;
  uint64_t* o_full = bars + 6;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 7);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nq = (a.S + 127) / 128;
  const int qb = nq - 1 - blockIdx.y;  // heavy (late) query blocks are scheduled first
  const int bh = blockIdx.x;
  const int b = bh / a.H, h = bh % a.H;
  const int m0 = qb * 128;
  const int nkv = a.causal ? (qb + 1) : nq;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    mbar_init(&k_full[0], 1);
    mbar_init(&k_full[1], 1);
    mbar_init(v_full, 1);
    mbar_init(s_full, 1);
    mbar_init(p_full, 128);
    mbar_init(o_full, 1);
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (EXPM != 0) {
    for (int i = threadIdx.x; i < 4096 / 4; i += ATT_THREADS)
      reinterpret_cast<uint32_t*>(sOnes)[i] = 0x3F803F80u;  // bf16 1.0 pairs
    fence_proxy_async_smem();
  }
  if (warp == 4) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
    tc_fence_before();
  }
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 4) {
    if (lane == 0) {
      constexpr uint32_t idesc_s = umma_idesc_bf16(128, 128, 0, 0);
      constexpr uint32_t idesc_o = umma_idesc_bf16(128, D, 0, 1);
      constexpr uint32_t idesc_l = umma_idesc_bf16(128, 16, 0, 0);
      auto load_tile = [&](uint8_t* dst, const CUtensorMap* tm, uint64_t* bar, int row0) {
        mbar_expect_tx(bar, TILE);
#pragma unroll
        for (int kd = 0; kd < NKD; ++kd) tma_load_4d(dst + kd * 16384, tm, bar, kd * 64, h, row0, b);
      };
      auto issue_s = [&](int stage) {
        const uint32_t aq = smem_u32(sQ), ak = smem_u32(sK + stage * TILE);
#pragma unroll
        for (int kd = 0; kd < NKD; ++kd)
#pragma unroll
          for (int k = 0; k < 4; ++k)
            umma_bf16_ss(tmem_base, umma_desc_sw128(aq + kd * 16384 + k * 32, 16, 1024),
                         umma_desc_sw128(ak + kd * 16384 + k * 32, 16, 1024), idesc_s,
                         (kd > 0 || k > 0) ? 1u : 0u);
        umma_commit(s_full);
      };
      bool ok = true;
      load_tile(sQ, &tmQ, q_full, m0);
      load_tile(sK, &tmK, &k_full[0], 0);
      load_tile(sV, &tmV, v_full, 0);
      if (nkv > 1) load_tile(sK + TILE, &tmK, &k_full[1], 128);
      ok = mbar_wait(q_full, 0, abort_flag) && mbar_wait(&k_full[0], 0, abort_flag);
      if (!ok) att_error(a.status, abort_flag, NKB_ERR_TMA_WAIT);
      if (ok) {
        tc_fence_after();
        issue_s(0);
      }
      for (int j = 0; j < nkv && ok; ++j) {
        const int st = j & 1;
        if (!mbar_wait(p_full, j & 1, abort_flag) || !mbar_wait(v_full, j & 1, abort_flag)) {
          att_error(a.status, abort_flag, NKB_ERR_ACC_WAIT);
          break;
        }
        tc_fence_after();
        {
          const uint32_t ap = smem_u32(sP), av = smem_u32(sV);
#pragma unroll
          for (int k = 0; k < 8; ++k)
            umma_bf16_ss(tmem_base + O_COL,
                         umma_desc_sw128(ap + (k >> 2) * 16384 + (k & 3) * 32, 16, 1024),
                         umma_desc_sw128(av + k * 2048, 16384, 1024), idesc_o, k > 0 ? 1u : 0u);
          if (EXPM != 0) {
            const uint32_t ao = smem_u32(sOnes);
#pragma unroll
            for (int k = 0; k < 8; ++k)
              umma_bf16_ss(tmem_base + L_COL,
                           umma_desc_sw128(ap + (k >> 2) * 16384 + (k & 3) * 32, 16, 1024),
                           umma_desc_sw128(ao + (k >> 2) * 2048 + (k & 3) * 32, 16, 1024),
                           idesc_l, k > 0 ? 1u : 0u);
          }
          umma_commit(o_full);
        }
        if (j + 1 < nkv) {
          if (!mbar_wait(&k_full[st ^ 1], ((j + 1) >> 1) & 1, abort_flag)) {
            att_error(a.status, abort_flag, NKB_ERR_TMA_WAIT);
            break;
          }
          tc_fence_after();
          issue_s(st ^ 1);
          // PV_j (and S_j) retired: V buffer and K[st] are free again
          if (!mbar_wait(o_full, j & 1, abort_flag)) {
            att_error(a.status, abort_flag, NKB_ERR_ACC_WAIT);
            break;
          }
          load_tile(sV, &tmV, v_full, (j + 1) * 128);
          if (j + 2 < nkv) load_tile(sK + st * TILE, &tmK, &k_full[st], (j + 2) * 128);
        }
      }
    }
  } else {
    // ------------------------------------------------------------- softmax
    const int r = warp * 32 + lane;
    const int qi = m0 + r;
    const uint32_t t_lane = tmem_base + (uint32_t(warp * 32) << 16);
    float m = -INFINITY, l = 0.f;
    float O[D];
#pragma unroll
    for (int i = 0; i < D; ++i) O[i] = 0.f;
    bool ok = true;
    for (int j = 0; j < nkv; ++j) {
      if (!mbar_wait(s_full, j & 1, abort_flag)) {
        att_error(a.status, abort_flag, NKB_ERR_ACC_WAIT);
        ok = false;
        break;
      }
      tc_fence_after();
      const bool need_mask = (j == nkv - 1) && (a.causal || (a.S & 127));
      const int kv0 = j * 128;
      // pass 1: row max
      float mx = -INFINITY;
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint32_t s[32];
        tmem_ld_32x32(t_lane + c * 32, s);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          float x = __uint_as_float(s[i]);
          if (need_mask) {
            const int kv = kv0 + c * 32 + i;
            if (kv >= a.S || (a.causal && kv > qi)) x = -INFINITY;
          }
          mx = fmaxf(mx, x);
        }
      }
      const float m_new = fmaxf(m, mx);
      const float alpha = exp2f((m - m_new) * a.scale_log2);
      // fold in the previous block's P V, then move the accumulator to the new max
      if (j > 0) {
        if (!mbar_wait(o_full, (j - 1) & 1, abort_flag)) {
          att_error(a.status, abort_flag, NKB_ERR_ACC_WAIT);
          ok = false;
          break;
        }
        tc_fence_after();
#pragma unroll
        for (int c = 0; c < D / 32; ++c) {
          uint32_t pv[32];
          tmem_ld_32x32(t_lane + O_COL + c * 32, pv);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) O[c * 32 + i] = (O[c * 32 + i] + __uint_as_float(pv[i])) * alpha;
        }
        if (EXPM != 0) {
          const float rs = __uint_as_float(tmem_ld_32x1(t_lane + L_COL));
          tmem_ld_wait();
          l = (l + rs) * alpha;
        }
      }
      // pass 2: probabilities -> shared memory (swizzled K-major A operand)
      float rowsum = 0.f;
      const float mneg = -m_new * a.scale_log2;
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint32_t s[32];
        tmem_ld_32x32(t_lane + c * 32, s);
        tmem_ld_wait();
        uint32_t pk[16];
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          float x0 = fmaf(__uint_as_float(s[i]), a.scale_log2, mneg);
          float x1 = fmaf(__uint_as_float(s[i + 1]), a.scale_log2, mneg);
          if (need_mask) {
            const int kv = kv0 + c * 32 + i;
            if (kv >= a.S || (a.causal && kv > qi)) x0 = -INFINITY;
            if (kv + 1 >= a.S || (a.causal && kv + 1 > qi)) x1 = -INFINITY;
          }
          if (EXPM == 0) {
            const float p0 = exp2f(x0), p1 = exp2f(x1);
            rowsum += p0 + p1;
            pk[i >> 1] = pack_bf16x2(p0, p1);
          } else if (EXPM == 1) {
            pk[i >> 1] = f16x2_to_bf16x2(ex2_f16x2(x0, x1));
          } else {
            pk[i >> 1] = ex2_bf16x2(x0, x1);
          }
        }
        uint8_t* base = sP + (c >> 1) * 16384;
#pragma unroll
        for (int q = 0; q < 4; ++q)
          *reinterpret_cast<uint4*>(base + sw128_off(r, (c & 1) * 4 + q)) =
              make_uint4(pk[4 * q], pk[4 * q + 1], pk[4 * q + 2], pk[4 * q + 3]);
      }
      if (EXPM == 0) l = l * alpha + rowsum;
      m = m_new;
      fence_proxy_async_smem();
      tc_fence_before();
      mbar_arrive(p_full);
    }
    if (ok && mbar_wait(o_full, (nkv - 1) & 1, abort_flag)) {
      tc_fence_after();
      if (EXPM != 0) {
        l += __uint_as_float(tmem_ld_32x1(t_lane + L_COL));
        tmem_ld_wait();
      }
      const float inv = 1.f / l;
      __nv_bfloat16* orow = a.o + (long long)b * a.ob + (long long)h * a.oh + (long long)qi * a.os;
#pragma unroll
      for (int c = 0; c < D / 32; ++c) {
        uint32_t pv[32];
        tmem_ld_32x32(t_lane + O_COL + c * 32, pv);
        tmem_ld_wait();
        if (qi < a.S) {
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            uint32_t w[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const int i = q * 8 + e * 2;
              w[e] = pack_bf16x2((O[c * 32 + i] + __uint_as_float(pv[i])) * inv,
                                 (O[c * 32 + i + 1] + __uint_as_float(pv[i + 1])) * inv);
            }
            *reinterpret_cast<uint4*>(orow + c * 32 + q * 8) = make_uint4(w[0], w[1], w[2], w[3]);
          }
        }
      }
      if (qi < a.S) a.lse[((long long)b * a.H + h) * a.S + qi] = m * a.scale + __logf(l);
    } else if (ok) {
      att_error(a.status, abort_flag, NKB_ERR_ACC_WAIT);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 4) {
    if (*abort_flag)
      for (int i = 0; i < 1000; ++i) __nanosleep(1000);
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

#include "attention_fwd_pp.cuh"

// ------------------------------------------------------------------ backward
struct AttnBwdArgs {
  const float* lse;
  const float* delta;
  float* dq_acc;            // [B,H,S,D] fp32, cleared by the delta kernel of the same call
  __nv_bfloat16* dk;
  __nv_bfloat16* dv;        // same strides as k / v
  int B, H, S;
  long long sb, sh, ss;
  float scale, scale_log2;
  int causal;
  int* status;
};

__device__ __forceinline__ void red_add_v4(float* p, float a, float b, float c, float d) {
  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(p), "f"(a), "f"(b), "f"(c),
               "f"(d)
               : "memory");
}

template <int D>
__global__ void __launch_bounds__(ATT_THREADS, 1)
attn_bwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmDO,
                const AttnBwdArgs a) {
  constexpr int TILE = 128 * D * 2;
  constexpr int NKD = D / 64;
  constexpr int STAGES = (D == 64) ? 2 : 1;
  constexpr uint32_t TMEM_COLS = 512;
  constexpr uint32_t S_COL = 0, DP_COL = 128, DV_COL = 256, DK_COL = 256 + D;
  constexpr uint32_t DQ_COL = (D == 64) ? 384 : 0;  // D=128: dQ reuses the S columns
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                              ~uintptr_t(1023));
  uint8_t* sK = smem;
  uint8_t* sV = sK + TILE;
  uint8_t* sQ = sV + TILE;                 // STAGES
  uint8_t* sDO = sQ + STAGES * TILE;       // STAGES
  uint8_t* sP = sDO + STAGES * TILE;       // 32 KB
  uint8_t* sDS = sP + 32768;               // 32 KB
  uint64_t* bars = reinterpret_cast<uint64_t*>(sDS + 32768);
  uint64_t* kv_full = bars + 0;
  uint64_t* qdo_full = bars + 1;  // [2]
  uint64_t* sdp_full = bars + 3;
  uint64_t* pds_full = bars + 4;
  uint64_t* dq_full = bars + 5;
  uint64_t* dq_done = bars + 6;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 7);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nq = (a.S + 127) / 128;
  const int j = blockIdx.y;  // key block; early key blocks have the most work and go first
  const int bh = blockIdx.x;
  const int b = bh / a.H, h = bh % a.H;
  const int i0 = a.causal ? j : 0;
  const int niter = nq - i0;

  if (threadIdx.x == 0) {
    mbar_init(kv_full, 1);
    mbar_init(&qdo_full[0], 1);
    mbar_init(&qdo_full[1], 1);
    mbar_init(sdp_full, 1);
    mbar_init(pds_full, 128);
    mbar_init(dq_full, 1);
    mbar_init(dq_done, 128);
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 4) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
    tc_fence_before();
  }
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 4) {
    if (lane == 0) {
      constexpr uint32_t idesc_s = umma_idesc_bf16(128, 128, 0, 0);   // S, dP: K-major x K-major
      constexpr uint32_t idesc_tt = umma_idesc_bf16(128, D, 1, 1);    // dV, dK: MN-major x MN-major
      constexpr uint32_t idesc_dq = umma_idesc_bf16(128, D, 0, 1);    // dQ: K-major x MN-major
      auto load_tile = [&](uint8_t* dst, const CUtensorMap* tm, uint64_t* bar, int row0) {
#pragma unroll
        for (int kd = 0; kd < NKD; ++kd) tma_load_4d(dst + kd * 16384, tm, bar, kd * 64, h, row0, b);
      };
      mbar_expect_tx(kv_full, 2 * TILE);
      load_tile(sK, &tmK, kv_full, j * 128);
      load_tile(sV, &tmV, kv_full, j * 128);
      for (int s = 0; s < STAGES && s < niter; ++s) {
        mbar_expect_tx(&qdo_full[s], 2 * TILE);
        load_tile(sQ + s * TILE, &tmQ, &qdo_full[s], (i0 + s) * 128);
        load_tile(sDO + s * TILE, &tmDO, &qdo_full[s], (i0 + s) * 128);
      }
      bool ok = mbar_wait(kv_full, 0, abort_flag);
      if (!ok) att_error(a.status, abort_flag, NKB_ERR_TMA_WAIT);
      for (int it = 0; it < niter && ok; ++it) {
        const int st = it % STAGES;
        if (!mbar_wait(&qdo_full[st], (it / STAGES) & 1, abort_flag)) {
          att_error(a.status, abort_flag, NKB_ERR_TMA_WAIT);
          break;
        }
        if (D == 128 && it > 0) {
          if (!mbar_wait(dq_done, (it - 1) & 1, abort_flag)) {
            att_error(a.status, abort_flag, NKB_ERR_ACC_FREE);
            break;
          }
        }
        tc_fence_after();
        const uint32_t aK = smem_u32(sK), aV = smem_u32(sV), aQ = smem_u32(sQ + st * TILE),
                       aDO = smem_u32(sDO + st * TILE), aP = smem_u32(sP), aDS = smem_u32(sDS);
        // S = Q K^T ; dP = dO V^T
#pragma unroll
        for (int kd = 0; kd < NKD; ++kd)
#pragma unroll
          for (int k = 0; k < 4; ++k)
            umma_bf16_ss(tmem_base + S_COL, umma_desc_sw128(aQ + kd * 16384 + k * 32, 16, 1024),
                         umma_desc_sw128(aK + kd * 16384 + k * 32, 16, 1024), idesc_s,
                         (kd > 0 || k > 0) ? 1u : 0u);
#pragma unroll
        for (int kd = 0; kd < NKD; ++kd)
#pragma unroll
          for (int k = 0; k < 4; ++k)
            umma_bf16_ss(tmem_base + DP_COL, umma_desc_sw128(aDO + kd * 16384 + k * 32, 16, 1024),
                         umma_desc_sw128(aV + kd * 16384 + k * 32, 16, 1024), idesc_s,
                         (kd > 0 || k > 0) ? 1u : 0u);
        umma_commit(sdp_full);
        if (!mbar_wait(pds_full, it & 1, abort_flag)) {
          att_error(a.status, abort_flag, NKB_ERR_ACC_WAIT);
          break;
        }
        tc_fence_after();
        // dV += P^T dO ; dK += dS^T Q  (contraction over the 128 queries)
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          umma_bf16_ss(tmem_base + DV_COL, umma_desc_sw128(aP + k * 2048, 16384, 1024),
                       umma_desc_sw128(aDO + k * 2048, 16384, 1024), idesc_tt,
                       (it > 0 || k > 0) ? 1u : 0u);
        }
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          umma_bf16_ss(tmem_base + DK_COL, umma_desc_sw128(aDS + k * 2048, 16384, 1024),
                       umma_desc_sw128(aQ + k * 2048, 16384, 1024), idesc_tt,
                       (it > 0 || k > 0) ? 1u : 0u);
        }
        // dQ = dS K  (contraction over the 128 keys)
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          umma_bf16_ss(tmem_base + DQ_COL,
                       umma_desc_sw128(aDS + (k >> 2) * 16384 + (k & 3) * 32, 16, 1024),
                       umma_desc_sw128(aK + k * 2048, 16384, 1024), idesc_dq, k > 0 ? 1u : 0u);
        }
        umma_commit(dq_full);
        if (it + STAGES < niter) {
          if (!mbar_wait(dq_full, it & 1, abort_flag)) {
            att_error(a.status, abort_flag, NKB_ERR_ACC_WAIT);
            break;
          }
          mbar_expect_tx(&qdo_full[st], 2 * TILE);
          load_tile(sQ + st * TILE, &tmQ, &qdo_full[st], (i0 + it + STAGES) * 128);
          load_tile(sDO + st * TILE, &tmDO, &qdo_full[st], (i0 + it + STAGES) * 128);
        }
      }
    }
  } else {
    const int r = warp * 32 + lane;
    const uint32_t t_lane = tmem_base + (uint32_t(warp * 32) << 16);
    const long long bh_off = ((long long)b * a.H + h) * a.S;
    bool ok = true;
    for (int it = 0; it < niter; ++it) {
      const int i = i0 + it;
      const int qi = i * 128 + r;
      float lse_r = 0.f, delta_r = 0.f;
      if (qi < a.S) {
        lse_r = a.lse[bh_off + qi] * LOG2E;
        delta_r = a.delta[bh_off + qi];
      }
      if (!mbar_wait(sdp_full, it & 1, abort_flag)) {
        att_error(a.status, abort_flag, NKB_ERR_ACC_WAIT);
        ok = false;
        break;
      }
      tc_fence_after();
      const bool need_mask = (a.causal && i == j) || (a.S & 127);
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint32_t s[32], dp[32];
        tmem_ld_32x32(t_lane + S_COL + c * 32, s);
        tmem_ld_32x32(t_lane + DP_COL + c * 32, dp);
        tmem_ld_wait();
        uint32_t pk[16], dk_[16];
#pragma unroll
        for (int e = 0; e < 32; e += 2) {
          float p0 = exp2f(fmaf(__uint_as_float(s[e]), a.scale_log2, -lse_r));
          float p1 = exp2f(fmaf(__uint_as_float(s[e + 1]), a.scale_log2, -lse_r));
          if (need_mask) {
            const int kv = j * 128 + c * 32 + e;
            if (qi >= a.S || kv >= a.S || (a.causal && kv > qi)) p0 = 0.f;
            if (qi >= a.S || kv + 1 >= a.S || (a.causal && kv + 1 > qi)) p1 = 0.f;
          }
          float d0 = p0 * (__uint_as_float(dp[e]) - delta_r) * a.scale;
          float d1 = p1 * (__uint_as_float(dp[e + 1]) - delta_r) * a.scale;
          pk[e >> 1] = pack_bf16x2(p0, p1);
          dk_[e >> 1] = pack_bf16x2(d0, d1);
        }
        const uint32_t tile_off = (c >> 1) * 16384;
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const uint32_t off = tile_off + sw128_off(r, (c & 1) * 4 + q);
          *reinterpret_cast<uint4*>(sP + off) =
              make_uint4(pk[4 * q], pk[4 * q + 1], pk[4 * q + 2], pk[4 * q + 3]);
          *reinterpret_cast<uint4*>(sDS + off) =
              make_uint4(dk_[4 * q], dk_[4 * q + 1], dk_[4 * q + 2], dk_[4 * q + 3]);
        }
      }
      fence_proxy_async_smem();
      tc_fence_before();
      mbar_arrive(pds_full);
      if (!mbar_wait(dq_full, it & 1, abort_flag)) {
        att_error(a.status, abort_flag, NKB_ERR_ACC_WAIT);
        ok = false;
        break;
      }
      tc_fence_after();
      float* dq_row = a.dq_acc + (bh_off + qi) * D;
#pragma unroll
      for (int c = 0; c < D / 32; ++c) {
        uint32_t v[32];
        tmem_ld_32x32(t_lane + DQ_COL + c * 32, v);
        tmem_ld_wait();
        if (qi < a.S) {
#pragma unroll
          for (int q = 0; q < 8; ++q)
            red_add_v4(dq_row + c * 32 + q * 4, __uint_as_float(v[4 * q]),
                       __uint_as_float(v[4 * q + 1]), __uint_as_float(v[4 * q + 2]),
                       __uint_as_float(v[4 * q + 3]));
        }
      }
      if (D == 128) {
        tc_fence_before();
        mbar_arrive(dq_done);
      }
    }
    if (ok && niter > 0) {
      // the last dq_full commit also covers the final dV / dK updates
      const int ki = j * 128 + r;
      const long long off = (long long)b * a.sb + (long long)h * a.sh + (long long)ki * a.ss;
#pragma unroll
      for (int which = 0; which < 2; ++which) {
        __nv_bfloat16* dst = (which == 0 ? a.dv : a.dk) + off;
        const uint32_t col = which == 0 ? DV_COL : DK_COL;
#pragma unroll
        for (int c = 0; c < D / 32; ++c) {
          uint32_t v[32];
          tmem_ld_32x32(t_lane + col + c * 32, v);
          tmem_ld_wait();
          if (ki < a.S) {
#pragma unroll
            for (int q = 0; q < 4; ++q)
              *reinterpret_cast<uint4*>(dst + c * 32 + q * 8) = make_uint4(
                  pack_bf16x2(__uint_as_float(v[8 * q]), __uint_as_float(v[8 * q + 1])),
                  pack_bf16x2(__uint_as_float(v[8 * q + 2]), __uint_as_float(v[8 * q + 3])),
                  pack_bf16x2(__uint_as_float(v[8 * q + 4]), __uint_as_float(v[8 * q + 5])),
                  pack_bf16x2(__uint_as_float(v[8 * q + 6]), __uint_as_float(v[8 * q + 7])));
          }
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 4) {
    if (*abort_flag)
      for (int i = 0; i < 1000; ++i) __nanosleep(1000);
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

#include "attention_bwd_pp.cuh"

// delta[b,h,s] = sum_d o * do ; 8 lanes per row, DELTA_ROWS rows per thread so that each
// thread has several independent 16-byte loads in flight
constexpr int DELTA_ROWS = 4;
__global__ void __launch_bounds__(256)
attn_delta_kernel(const __nv_bfloat16* __restrict__ o, const __nv_bfloat16* __restrict__ dout,
                  float* __restrict__ delta, int B, int H, int S, int D, long long ob, long long oh,
                  long long os, float* __restrict__ dq_acc) {
  // also clears the fp32 dQ accumulator [B*H*S, D] (each lane its D/8 floats of the row), so no
  // separate fill kernel runs before the backward kernel
  const long long slot = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 3;
  const int sub = threadIdx.x & 7;
  const long long total = (long long)B * H * S;
  const long long nslots = (long long)gridDim.x * (blockDim.x >> 3);
  float acc[DELTA_ROWS];
  uint4 xs[DELTA_ROWS], ys[DELTA_ROWS];
  if (D == 64) {
    // one 16-byte piece of o and of dout per lane and row: issue all loads, then reduce
#pragma unroll
    for (int u = 0; u < DELTA_ROWS; ++u) {
      const long long row = slot + u * nslots;
      xs[u] = ys[u] = make_uint4(0, 0, 0, 0);
      if (row < total) {
        // slots walk (b, s, h): neighbouring slots read neighbouring heads of one token, i.e.
        // contiguous memory of the [B, S, H*D] tensors
        const int h = (int)(row % H);
        const int s = (int)((row / H) % S);
        const int b = (int)(row / ((long long)S * H));
        const long long off = (long long)b * ob + (long long)h * oh + (long long)s * os + sub * 8;
        xs[u] = ld_nc_v4(o + off);
        ys[u] = ld_nc_v4(dout + off);
      }
    }
#pragma unroll
    for (int u = 0; u < DELTA_ROWS; ++u) {
      const uint32_t xu[4] = {xs[u].x, xs[u].y, xs[u].z, xs[u].w};
      const uint32_t yu[4] = {ys[u].x, ys[u].y, ys[u].z, ys[u].w};
      acc[u] = 0.f;
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const float2 f = unpack_bf16x2(xu[q]), g = unpack_bf16x2(yu[q]);
        acc[u] += f.x * g.x + f.y * g.y;
      }
    }
  } else {
#pragma unroll
    for (int u = 0; u < DELTA_ROWS; ++u) {
      const long long row = slot + u * nslots;
      acc[u] = 0.f;
      if (row < total) {
        // slots walk (b, s, h): neighbouring slots read neighbouring heads of one token, i.e.
        // contiguous memory of the [B, S, H*D] tensors
        const int h = (int)(row % H);
        const int s = (int)((row / H) % S);
        const int b = (int)(row / ((long long)S * H));
        const long long off = (long long)b * ob + (long long)h * oh + (long long)s * os;
        for (int d = sub * 8; d < D; d += 64) {
          const uint4 x = ld_nc_v4(o + off + d);
          const uint4 y = ld_nc_v4(dout + off + d);
          const uint32_t xu[4] = {x.x, x.y, x.z, x.w}, yu[4] = {y.x, y.y, y.z, y.w};
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            const float2 f = unpack_bf16x2(xu[q]), g = unpack_bf16x2(yu[q]);
            acc[u] += f.x * g.x + f.y * g.y;
          }
        }
      }
    }
  }
#pragma unroll
  for (int u = 0; u < DELTA_ROWS; ++u) {
    float a = acc[u];
    a += __shfl_xor_sync(0xffffffffu, a, 1);
    a += __shfl_xor_sync(0xffffffffu, a, 2);
    a += __shfl_xor_sync(0xffffffffu, a, 4);
    const long long row = slot + u * nslots;
    const long long orow = row < total
        ? ((row / ((long long)S * H)) * H + row % H) * S + (row / H) % S : 0;  // (b*H + h)*S + s
    if (row < total && sub == 0) delta[orow] = a;
    if (dq_acc && row < total) {
      float4* z = reinterpret_cast<float4*>(dq_acc + orow * D + sub * (D / 8));
      for (int i = 0; i < D / 32; ++i) z[i] = make_float4(0.f, 0.f, 0.f, 0.f);
    }
  }
}

// dq (bf16, strided) <- dq_acc (fp32 [B,H,S,D])
__global__ void __launch_bounds__(256)
attn_dq_convert_kernel(const float* __restrict__ acc, __nv_bfloat16* __restrict__ dq, int B, int H,
                       int S, int D, long long sb, long long sh, long long ss) {
  const long long n8 = (long long)B * H * S * D / 8;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n8;
       i += (long long)gridDim.x * blockDim.x) {
    const long long e = i * 8;
    const int d = (int)(e % D);
    const long long row = e / D;
    const int s = (int)(row % S);
    const int h = (int)((row / S) % H);
    const int b = (int)(row / ((long long)S * H));
    float4 x = reinterpret_cast<const float4*>(acc)[i * 2];
    float4 y = reinterpret_cast<const float4*>(acc)[i * 2 + 1];
    *reinterpret_cast<uint4*>(dq + (long long)b * sb + (long long)h * sh + (long long)s * ss + d) =
        make_uint4(pack_bf16x2(x.x, x.y), pack_bf16x2(x.z, x.w), pack_bf16x2(y.x, y.y),
                   pack_bf16x2(y.z, y.w));
  }
}

// ------------------------------------------------------------------ host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn att_encode_fn() {
  // The encode call is a driver-API entry and needs the primary context current on the calling
  // thread; a thread that has made no runtime call yet (e.g. an autograd worker whose first
  // work is this library) has none, so bind it once per thread.
  static thread_local bool ctx_bound = false;
  if (!ctx_bound) {
    cudaFree(nullptr);
    ctx_bound = true;
  }
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) ==
            cudaSuccess && q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

// [B, S, H, D] view with element strides (sb, ss, sh, 1); box = 64 (d) x 1 (h) x 128 (s) x 1 (b)
static int make_tmap_bshd(CUtensorMap* out, const void* base, int B, int H, int S, int D,
                          long long sb, long long sh, long long ss) {
  EncodeTiledFn fn = att_encode_fn();
  if (!fn) return -1;
  if ((sb & 7) || (sh & 7) || (ss & 7) || (reinterpret_cast<uintptr_t>(base) & 15)) return -3;
  cuuint64_t gdim[4] = {(cuuint64_t)D, (cuuint64_t)H, (cuuint64_t)S, (cuuint64_t)B};
  cuuint64_t gstride[3] = {(cuuint64_t)sh * 2, (cuuint64_t)ss * 2, (cuuint64_t)sb * 2};
  cuuint32_t box[4] = {64, 1, 128, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(base), gdim, gstride,
                  box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -(int)r - 1000;
}

// 0: fp32 exp (default; the packed forms measured no faster: the softmax warps are not
// bound by the exponential alone), 1: packed f16x2, 2: packed bf16x2
static int g_attn_exp_mode = 0;

template <int D, int EXPM>
static int launch_fwd(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv,
                      const AttnFwdArgs& a, cudaStream_t s) {
  constexpr int smem = 4 * (128 * D * 2) + 32768 + 4096 + 1024 + 128;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attn_fwd_kernel<D, EXPM>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  dim3 grid(a.B * a.H, (a.S + 127) / 128);
  attn_fwd_kernel<D, EXPM><<<grid, ATT_THREADS, smem, s>>>(tq, tk, tv, a);
  return (int)cudaGetLastError();
}

// 1: ping-pong kernel (two query tiles per CTA, P through TMEM), 0: one query tile per CTA
static int g_attn_fwd_impl = 1;

template <int D, int EXPM>
static int launch_fwd_pp(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv,
                         const AttnFwdArgs& a, cudaStream_t s) {
  constexpr int smem = 6 * (128 * D * 2) + 1024 + 256;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attn_fwd_pp_kernel<D, EXPM>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  dim3 grid(a.B * a.H, (a.S + 255) / 256);
  attn_fwd_pp_kernel<D, EXPM><<<grid, ATT2_THREADS, smem, s>>>(tq, tk, tv, a);
  return (int)cudaGetLastError();
}

template <int D>
static int launch_fwd_mode(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv,
                           const AttnFwdArgs& a, cudaStream_t s) {
  if (g_attn_fwd_impl == 1) {
    if (g_attn_exp_mode == 0) return launch_fwd_pp<D, 0>(tq, tk, tv, a, s);
    return launch_fwd_pp<D, 1>(tq, tk, tv, a, s);
  }
  if (g_attn_exp_mode == 0) return launch_fwd<D, 0>(tq, tk, tv, a, s);
  if (g_attn_exp_mode == 2) return launch_fwd<D, 2>(tq, tk, tv, a, s);
  return launch_fwd<D, 1>(tq, tk, tv, a, s);
}

template <int D>
static int launch_bwd(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv,
                      const CUtensorMap& tdo, const AttnBwdArgs& a, cudaStream_t s) {
  constexpr int STAGES = (D == 64) ? 2 : 1;
  constexpr int smem = (2 + 2 * STAGES) * (128 * D * 2) + 65536 + 1024 + 128;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attn_bwd_kernel<D>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  dim3 grid(a.B * a.H, (a.S + 127) / 128);
  attn_bwd_kernel<D><<<grid, ATT_THREADS, smem, s>>>(tq, tk, tv, tdo, a);
  return (int)cudaGetLastError();
}

// fp32 dQ accumulator [B*H, S, D] as a 3-D map; box = 32 (d) x 128 (s) x 1, 128B swizzle
static int make_tmap_dq(CUtensorMap* out, float* base, int BH, int S, int D) {
  EncodeTiledFn fn = att_encode_fn();
  if (!fn) return -1;
  if (reinterpret_cast<uintptr_t>(base) & 15) return -3;
  cuuint64_t gdim[3] = {(cuuint64_t)D, (cuuint64_t)S, (cuuint64_t)BH};
  cuuint64_t gstride[2] = {(cuuint64_t)D * 4, (cuuint64_t)S * D * 4};
  cuuint32_t box[3] = {32, 128, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, base, gdim, gstride, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -(int)r - 1000;
}

// 1: warp-specialised kernel (head dim 64), 0: serial kernel
static int g_attn_bwd_impl = 1;

static int launch_bwd_pp(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv,
                         const CUtensorMap& tdo, const CUtensorMap& tdq, const AttnBwdArgs& a,
                         cudaStream_t s) {
  constexpr int smem = AttnBwd2Smem::BYTES;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attn_bwd_pp_kernel,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  dim3 grid(a.B * a.H, (a.S + 127) / 128);
  attn_bwd_pp_kernel<<<grid, BWD2_THREADS, smem, s>>>(tq, tk, tv, tdo, tdq, a);
  return (int)cudaGetLastError();
}

}  // namespace nkb

using namespace nkb;

extern "C" void nkb_attn_set_bwd_impl(int impl) { nkb::g_attn_bwd_impl = impl; }

// 0 = fp32 exponentials (default), 1 = packed half, 2 = packed bf16 (one-tile kernel only)
extern "C" void nkb_attn_set_exp_mode(int mode) { nkb::g_attn_exp_mode = mode; }
// 1 = ping-pong forward kernel (default), 0 = one query tile per CTA
extern "C" void nkb_attn_set_fwd_impl(int impl) { nkb::g_attn_fwd_impl = impl; }

extern "C" int nkb_attn_fwd(const void* q, const void* k, const void* v, void* o, float* lse,
                            int B, int H, int S, int D, long long sb, long long sh, long long ss,
                            long long ob, long long oh, long long os, float scale, int causal,
                            int* status, void* stream) {
  if (D != 64 && D != 128) return -5;
  if ((ob & 7) || (oh & 7) || (os & 7) || (reinterpret_cast<uintptr_t>(o) & 15)) return -3;
  CUtensorMap tq, tk, tv;
  int rc;
  if ((rc = make_tmap_bshd(&tq, q, B, H, S, D, sb, sh, ss))) return rc;
  if ((rc = make_tmap_bshd(&tk, k, B, H, S, D, sb, sh, ss))) return rc;
  if ((rc = make_tmap_bshd(&tv, v, B, H, S, D, sb, sh, ss))) return rc;
  AttnFwdArgs a;
  a.o = static_cast<__nv_bfloat16*>(o);
  a.lse = lse;
  a.B = B; a.H = H; a.S = S;
  a.ob = ob; a.oh = oh; a.os = os;
  a.scale = scale;
  a.scale_log2 = scale * LOG2E;
  a.causal = causal;
  a.status = status;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  return D == 64 ? launch_fwd_mode<64>(tq, tk, tv, a, s) : launch_fwd_mode<128>(tq, tk, tv, a, s);
}

extern "C" int nkb_attn_bwd(const void* q, const void* k, const void* v, const void* o,
                            const void* dout, const float* lse, void* dq, void* dk, void* dv,
                            float* delta, float* dq_acc, int B, int H, int S, int D, long long sb,
                            long long sh, long long ss, long long ob, long long oh, long long os,
                            float scale, int causal, int* status, void* stream) {
  if (D != 64 && D != 128) return -5;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  CUtensorMap tq, tk, tv, tdo;
  int rc;
  if ((rc = make_tmap_bshd(&tq, q, B, H, S, D, sb, sh, ss))) return rc;
  if ((rc = make_tmap_bshd(&tk, k, B, H, S, D, sb, sh, ss))) return rc;
  if ((rc = make_tmap_bshd(&tv, v, B, H, S, D, sb, sh, ss))) return rc;
  if ((rc = make_tmap_bshd(&tdo, dout, B, H, S, D, ob, oh, os))) return rc;
  const long long rows = (long long)B * H * S;
  attn_delta_kernel<<<(unsigned)((rows * 8 + 256 * DELTA_ROWS - 1) / (256 * DELTA_ROWS)), 256, 0, s>>>(
      static_cast<const __nv_bfloat16*>(o), static_cast<const __nv_bfloat16*>(dout), delta, B, H, S,
      D, ob, oh, os, dq_acc);
  AttnBwdArgs a;
  a.lse = lse; a.delta = delta; a.dq_acc = dq_acc;
  a.dk = static_cast<__nv_bfloat16*>(dk);
  a.dv = static_cast<__nv_bfloat16*>(dv);
  a.B = B; a.H = H; a.S = S;
  a.sb = sb; a.sh = sh; a.ss = ss;
  a.scale = scale;
  a.scale_log2 = scale * LOG2E;
  a.causal = causal;
  a.status = status;
  if (D == 64 && g_attn_bwd_impl >= 1) {
    CUtensorMap tdq;
    if ((rc = make_tmap_dq(&tdq, dq_acc, B * H, S, D))) return rc;
    rc = launch_bwd_pp(tq, tk, tv, tdo, tdq, a, s);
  } else {
    rc = D == 64 ? launch_bwd<64>(tq, tk, tv, tdo, a, s) : launch_bwd<128>(tq, tk, tv, tdo, a, s);
  }
  if (rc) return rc;
  long long n8 = rows * D / 8;
  int blocks = (int)((n8 + 255) / 256);
  if (blocks > 148 * 8) blocks = 148 * 8;
  attn_dq_convert_kernel<<<blocks, 256, 0, s>>>(dq_acc, static_cast<__nv_bfloat16*>(dq), B, H, S, D,
                                                sb, sh, ss);
  return (int)cudaGetLastError();
}

NKB_DEFINE_WAIT_SETTER(attn)
