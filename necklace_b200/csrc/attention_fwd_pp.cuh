// Ping-pong flash-attention forward for sm_100a (included by attention_sm100.cu inside
// namespace nkb).
//
// One CTA per (256-query block, batch*head), one CTA per SM.  Two softmax warpgroups
// (warps 0-3: query rows 0..127 of the block, warps 4-7: rows 128..255) share every
// K / V tile; warp 8 issues the TMA loads, warps 9 and 10 the tcgen05.mma instructions of
// one half each (an issuing thread blocks while the tensor pipe is busy and every
// barrier probe costs ~50 cycles, so one thread for both halves was the bottleneck);
// the control warpgroup hands most of its registers to the softmax warpgroups.
// While one warpgroup runs its softmax the tensor cores work for the other one, so the
// exponential unit, not the dependency chain S -> softmax -> PV, sets the pace.
//
//   TMEM columns: S_a [0,128)  S_b [128,256)  O_a [256,256+D)  O_b [256+D,256+2D)
//                 and for D = 64: P_a [384,448)  P_b [448,512)
//   * S = Q K^T lands in TMEM; a thread owns one query row (TMEM lane) and reads all
//     128 scores of the key block at once.
//   * P (bf16 pairs) goes back to TMEM and is the A operand of the P V MMA straight from
//     there: no shared-memory staging.  With D = 64 it has columns of its own, so the
//     next S of a warpgroup is issued as soon as the warpgroup has read the current one
//     and is ready before the softmax of the current block ends; with D = 128 TMEM is
//     full, P overwrites the first 64 columns of its S buffer and the next S follows
//     the P V MMA.
//   * O accumulates in TMEM across key blocks.  The running maximum is only moved (and
//     O rescaled through tcgen05.ld / st) when it grew by more than 2^8 since the last
//     move; until then probabilities are taken against the older maximum, which keeps
//     them below 256 and leaves the result unchanged after the final division.
//   * EXPM 0: fp32 ex2 per element; EXPM 1: packed half ex2 (two per MUFU op).
//
// All waits are bounded; a failed wait sets the status word and the abort flag.
// The reference has no attention layer.
#pragma once

constexpr int ATT2_THREADS = 384;
// setmaxnreg budget: the CTA owns threads x 168 registers (the compile-time cap)
static_assert(128 * 40 + 256 * 232 <= ATT2_THREADS * 168, "register budget");


template <int D, int EXPM>
__global__ void __launch_bounds__(ATT2_THREADS, 1)
attn_fwd_pp_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                   const __grid_constant__ CUtensorMap tmV, const AttnFwdArgs a) {
  constexpr int TILE = 128 * D * 2;  // bytes of a 128 x D bf16 tile
  constexpr int NKD = D / 64;        // 64-wide sub-tiles along the head dim
  constexpr uint32_t TMEM_COLS = 512;
  constexpr uint32_t O_COL = 256;
  constexpr bool PSEP = (D == 64);  // P has TMEM columns of its own
  constexpr uint32_t P_COL = 384;
  constexpr float RESCALE_LOG2 = 8.f;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                              ~uintptr_t(1023));
  uint8_t* sQ = smem;             // two query tiles
  uint8_t* sK = sQ + 2 * TILE;    // two stages
  uint8_t* sV = sK + 2 * TILE;    // two stages
  uint64_t* bars = reinterpret_cast<uint64_t*>(sV + 2 * TILE);
  uint64_t* q_full = bars + 0;
  uint64_t* k_full = bars + 1;    // [2]
  uint64_t* v_full = bars + 3;    // [2]
  uint64_t* k_empty = bars + 5;   // [2]
  uint64_t* v_empty = bars + 7;   // [2]
  uint64_t* s_full = bars + 9;    // [2] one per warpgroup
  uint64_t* p_full = bars + 11;   // [2]
  uint64_t* p_free = bars + 13;   // [2] P V of a block retired: O stable, P columns free
  uint64_t* s_free = bars + 15;   // [2] S read into registers (D = 64)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 17);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nq2 = (a.S + 255) / 256;
  const int qb = nq2 - 1 - blockIdx.y;  // heavy (late) query blocks are scheduled first
  const int bh = blockIdx.x;
  const int b = bh / a.H, h = bh % a.H;
  const int m0 = qb * 256;
  const int nkv_all = (a.S + 127) / 128;
  // key blocks each half of the query block attends to
  const int n0 = a.causal ? min(nkv_all, 2 * qb + 1) : nkv_all;
  const int n1 = (m0 + 128 < a.S) ? (a.causal ? min(nkv_all, 2 * qb + 2) : nkv_all) : 0;
  const int nmax = max(n0, n1);

  // The TMA thread sets up the barriers and puts the first loads (Q, two K / V stages) in
  // flight before the CTA-wide sync, so they overlap the TMEM allocation and the sync.
  auto load_tile = [&](uint8_t* dst, const CUtensorMap* tm, uint64_t* bar, int row0) {
#pragma unroll
    for (int kd = 0; kd < NKD; ++kd) tma_load_4d(dst + kd * 16384, tm, bar, kd * 64, h, row0, b);
  };
  if (threadIdx.x == 256) {
    mbar_init(q_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&k_full[i], 1);
      mbar_init(&v_full[i], 1);
      mbar_init(&k_empty[i], n1 > 0 ? 2 : 1);  // one commit per active half
      mbar_init(&v_empty[i], n1 > 0 ? 2 : 1);
      mbar_init(&s_full[i], 1);
      mbar_init(&p_full[i], 4);  // one arrival per softmax warp
      mbar_init(&p_free[i], 1);
      mbar_init(&s_free[i], 4);
    }
    *abort_flag = 0;
    mbar_fence_init();
    mbar_expect_tx(q_full, 2 * TILE);
    load_tile(sQ, &tmQ, q_full, m0);
    load_tile(sQ + TILE, &tmQ, q_full, m0 + 128);
    for (int j = 0; j < 2 && j < nmax; ++j) {
      mbar_expect_tx(&k_full[j], TILE);
      load_tile(sK + j * TILE, &tmK, &k_full[j], j * 128);
      mbar_expect_tx(&v_full[j], TILE);
      load_tile(sV + j * TILE, &tmV, &v_full[j], j * 128);
    }
  }
  if (warp == 9) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
    tc_fence_before();
  }
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp >= 8) reg_alloc_dec<40>();
  if (warp == 8) {
    // ---------------------------------------------------------------- TMA producer
    if (lane == 0) {
      for (int j = 2; j < nmax; ++j) {  // stages 0 and 1 were filled before the sync
        const int st = j & 1;
        const uint32_t par = ((j >> 1) & 1) ^ 1;
        if (!mbar_wait(&k_empty[st], par, abort_flag)) {
          att_error(a.status, abort_flag, NKB_ERR_EMPTY_WAIT);
          break;
        }
        mbar_expect_tx(&k_full[st], TILE);
        load_tile(sK + st * TILE, &tmK, &k_full[st], j * 128);
        if (!mbar_wait(&v_empty[st], par, abort_flag)) {
          att_error(a.status, abort_flag, NKB_ERR_EMPTY_WAIT);
          break;
        }
        mbar_expect_tx(&v_full[st], TILE);
        load_tile(sV + st * TILE, &tmV, &v_full[st], j * 128);
      }
    }
  } else if (warp == 9 || warp == 10) {
    // ------------------------------------------------- MMA issuer of half x = warp - 9
    const int x = warp - 9;
    const int nx = x ? n1 : n0;
    if (lane == 0 && nx > 0) {
      constexpr uint32_t idesc_s = umma_idesc_bf16(128, 128, 0, 0);
      constexpr uint32_t idesc_o = umma_idesc_bf16(128, D, 0, 1);
      // descriptors are built once; per MMA only the start-address field (16-byte units) moves
      const uint64_t dq = umma_desc_sw128(smem_u32(sQ + x * TILE), 16, 1024);
      const uint64_t dK0 = umma_desc_sw128(smem_u32(sK), 16, 1024);
      const uint64_t dV0 = umma_desc_sw128(smem_u32(sV), 16384, 1024);
      const uint32_t t_sx = tmem_base + x * 128, t_ox = tmem_base + O_COL + x * D;
      const uint32_t t_px = tmem_base + (PSEP ? P_COL + x * 64 : x * 128);
      bool ok = true;
      auto wait_or_fail = [&](uint64_t* bar, uint32_t parity, int code) {
        if (ok && !mbar_wait(bar, parity, abort_flag)) {
          att_error(a.status, abort_flag, code);
          ok = false;
        }
      };
      // S of block j (K stage j & 1), then its commits
      auto issue_s = [&](int j) {
        wait_or_fail(&k_full[j & 1], (j >> 1) & 1, NKB_ERR_TMA_WAIT);
        if (!ok) return;
        tc_fence_after();
        const uint64_t dk = dK0 + (uint32_t)(j & 1) * (TILE >> 4);
#pragma unroll
        for (int kd = 0; kd < NKD; ++kd)
#pragma unroll
          for (int k = 0; k < 4; ++k)
            umma_bf16_ss(t_sx, dq + (kd * 1024 + k * 2), dk + (kd * 1024 + k * 2), idesc_s,
                         (kd > 0 || k > 0) ? 1u : 0u);
        umma_commit(&s_full[x]);
        umma_commit(&k_empty[j & 1]);
      };
      auto issue_pv = [&](int j) {
        wait_or_fail(&p_full[x], j & 1, NKB_ERR_ACC_WAIT);
        wait_or_fail(&v_full[j & 1], (j >> 1) & 1, NKB_ERR_TMA_WAIT);
        if (!ok) return;
        tc_fence_after();
        const uint64_t dv = dV0 + (uint32_t)(j & 1) * (TILE >> 4);
#pragma unroll
        for (int k = 0; k < 8; ++k)  // 16 keys per MMA: 8 TMEM columns of bf16 pairs
          umma_bf16_ts(t_ox, t_px + k * 8, dv + k * 128, idesc_o, (j > 0 || k > 0) ? 1u : 0u);
        umma_commit(&p_free[x]);
        umma_commit(&v_empty[j & 1]);
      };
      wait_or_fail(q_full, 0, NKB_ERR_TMA_WAIT);
      issue_s(0);
      for (int j = 0; j < nx && ok; ++j) {
        if (PSEP) {
          // the next S goes out as soon as the warpgroup has read the current one
          if (j + 1 < nx) {
            wait_or_fail(&s_free[x], j & 1, NKB_ERR_ACC_FREE);
            issue_s(j + 1);
          }
          issue_pv(j);
        } else {
          issue_pv(j);  // P overwrites S: the next S follows the P V that reads it
          if (j + 1 < nx) issue_s(j + 1);
        }
      }
    }
  } else if (warp < 8) {
    // --------------------------------------------------------------------- softmax
    reg_alloc_inc<232>();
    const int x = warp >> 2;                 // which half of the query block
    const int r = (warp & 3) * 32 + lane;    // row inside the 128-row tile (TMEM lane)
    const int qi = m0 + x * 128 + r;
    const uint32_t t_lane = tmem_base + (uint32_t((warp & 3) * 32) << 16);
    const uint32_t t_s = t_lane + x * 128;
    const uint32_t t_o = t_lane + O_COL + x * D;
    const uint32_t t_p = PSEP ? t_lane + P_COL + x * 64 : t_s;
    const int nkv = x ? n1 : n0;
    float m_ref = 0.f, l = 0.f;
    bool ok = true;
    for (int j = 0; j < nkv; ++j) {
      if (!mbar_wait(&s_full[x], j & 1, abort_flag)) {
        att_error(a.status, abort_flag, NKB_ERR_ACC_WAIT);
        ok = false;
        break;
      }
      tc_fence_after();
      uint32_t s[128];
#pragma unroll
      for (int c = 0; c < 4; ++c) tmem_ld_32x32(t_s + c * 32, s + c * 32);
      tmem_ld_wait();
      if (PSEP) {
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&s_free[x]);
      }
      const int kv0 = j * 128;
      const bool need_mask = (a.causal && kv0 + 127 > m0 + x * 128) || (kv0 + 128 > a.S);
      if (need_mask) {
#pragma unroll
        for (int i = 0; i < 128; ++i) {
          const int kv = kv0 + i;
          if (kv >= a.S || (a.causal && kv > qi)) s[i] = 0xFF800000u;  // -inf
        }
      }
      float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
      for (int i = 0; i < 128; i += 4) {
        mx0 = max3_f32(mx0, __uint_as_float(s[i]), __uint_as_float(s[i + 1]));
        mx1 = max3_f32(mx1, __uint_as_float(s[i + 2]), __uint_as_float(s[i + 3]));
      }
      const float mx = fmaxf(mx0, mx1);
      // P V of block j-1 must have retired before O is rescaled or P overwritten; the wait
      // sits as late as possible (after the exponentials unless O has to be rescaled)
      bool pv_done = (j == 0);
      auto wait_pv = [&]() -> bool {
        if (pv_done) return true;
        if (!mbar_wait(&p_free[x], (j - 1) & 1, abort_flag)) {
          att_error(a.status, abort_flag, NKB_ERR_ACC_WAIT);
          return false;
        }
        tc_fence_after();
        pv_done = true;
        return true;
      };
      if (j == 0) {
        m_ref = (mx == -INFINITY) ? 0.f : mx;
      } else {
        const bool grow = (mx - m_ref) * a.scale_log2 > RESCALE_LOG2;
        if (__any_sync(0xffffffffu, grow)) {
          if (!wait_pv()) {
            ok = false;
            break;
          }
          const float alpha = grow ? ex2_f32((m_ref - mx) * a.scale_log2) : 1.f;
          l *= alpha;
#pragma unroll
          for (int c = 0; c < D / 32; ++c) {
            uint32_t o[32];
            tmem_ld_32x32(t_o + c * 32, o);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
            tmem_st_32x16(t_o + c * 32, o);
            tmem_st_32x16(t_o + c * 32 + 16, o + 16);
          }
          if (grow) m_ref = mx;
        }
      }
      const float mneg = -m_ref * a.scale_log2;
      float sum0 = 0.f, sum1 = 0.f, sum2 = 0.f, sum3 = 0.f;
      uint32_t pk[64];
#pragma unroll
      for (int i = 0; i < 128; i += 4) {
        const float x0 = fmaf(__uint_as_float(s[i]), a.scale_log2, mneg);
        const float x1 = fmaf(__uint_as_float(s[i + 1]), a.scale_log2, mneg);
        const float x2 = fmaf(__uint_as_float(s[i + 2]), a.scale_log2, mneg);
        const float x3 = fmaf(__uint_as_float(s[i + 3]), a.scale_log2, mneg);
        float p0, p1, p2, p3;
        if (EXPM == 0) {
          p0 = ex2_f32(x0);
          p1 = ex2_f32(x1);
          p2 = ex2_f32(x2);
          p3 = ex2_f32(x3);
        } else {
          unpack_f16x2(ex2_f16x2(x0, x1), p0, p1);
          unpack_f16x2(ex2_f16x2(x2, x3), p2, p3);
        }
        sum0 += p0;
        sum1 += p1;
        sum2 += p2;
        sum3 += p3;
        pk[i >> 1] = pack_bf16x2(p0, p1);
        pk[(i >> 1) + 1] = pack_bf16x2(p2, p3);
      }
      if (!wait_pv()) {
        ok = false;
        break;
      }
#pragma unroll
      for (int c = 0; c < 4; ++c) tmem_st_32x16(t_p + c * 16, pk + c * 16);
      sum0 += sum2;
      sum1 += sum3;
      l += sum0 + sum1;
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_full[x]);
    }
    if (nkv > 0) {
      if (ok && mbar_wait(&p_free[x], (nkv - 1) & 1, abort_flag)) {
        tc_fence_after();
        const float inv = 1.f / l;
        __nv_bfloat16* orow =
            a.o + (long long)b * a.ob + (long long)h * a.oh + (long long)qi * a.os;
#pragma unroll
        for (int c = 0; c < D / 32; ++c) {
          uint32_t pv[32];
          tmem_ld_32x32(t_o + c * 32, pv);
          tmem_ld_wait();
          if (qi < a.S) {
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              uint32_t w[4];
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                const int i = q * 8 + e * 2;
                w[e] = pack_bf16x2(__uint_as_float(pv[i]) * inv, __uint_as_float(pv[i + 1]) * inv);
              }
              *reinterpret_cast<uint4*>(orow + c * 32 + q * 8) = make_uint4(w[0], w[1], w[2], w[3]);
            }
          }
        }
        if (qi < a.S) a.lse[((long long)b * a.H + h) * a.S + qi] = m_ref * a.scale + __logf(l);
      } else if (ok) {
        att_error(a.status, abort_flag, NKB_ERR_ACC_WAIT);
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 9) {
    if (*abort_flag)
      for (int i = 0; i < 1000; ++i) __nanosleep(1000);
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}
