// Warp-specialised flash-attention backward for sm_100a, head dim 64 (included by
// attention_sm100.cu inside namespace nkb).
//
// One CTA per (128-key block, batch*head) looping over query blocks, 16 warps:
//   warps 0-7   two compute warpgroups.  Scores are produced transposed (S^T = K Q^T,
//               dP^T = V dO^T), so a thread owns one KEY row (TMEM lane); warpgroup w takes
//               query columns [64w, 64w+64).  It forms P^T = exp2(S^T c - lse) and
//               dS^T = P^T (dP^T - delta), writes both back to TMEM as bf16 pairs (the A
//               operands of dV += P^T dO and dK += dS^T Q, read straight from TMEM) and
//               dS^T to shared memory (A operand of dQ = dS K, M = query contiguous).
//   warps 8-11  dQ writer: TMEM -> registers -> swizzled fp32 tile in shared memory ->
//               one TMA reduce-add into the fp32 dQ accumulator (no per-thread atomics).
//   warp 12     TMA producer (K, V once; Q, dO double-buffered).
//   warp 13     tcgen05.mma issuer.  dQ of block i-1 is issued behind S^T / dP^T of block
//               i, so it runs while the compute warpgroups work on block i.
//   warps 14-15 idle (they complete the fourth warpgroup for setmaxnreg).
//
//   TMEM columns: S^T [0,128) (P^T of warpgroup w over [64w, 64w+32))
//                 dP^T [128,256) (dS^T likewise)  dV [256,320)  dK [320,384)  dQ [384,448)
//
// lse / delta of the query block are staged in shared memory (they index columns here),
// fetched one block ahead.  All waits are bounded.  The reference has no attention layer.
#pragma once

constexpr int BWD2_THREADS = 512;
// setmaxnreg budget: the CTA owns threads x 128 registers (the compile-time cap)
static_assert(256 * 184 + 128 * 88 + 128 * 40 <= BWD2_THREADS * 128, "register budget");

struct AttnBwd2Smem {
  static constexpr int TILE = 128 * 64 * 2;      // 16 KB bf16 tile
  static constexpr int K_OFF = 0;
  static constexpr int V_OFF = TILE;
  static constexpr int Q_OFF = 2 * TILE;          // 2 stages
  static constexpr int DO_OFF = 4 * TILE;         // 2 stages
  static constexpr int DS_OFF = 6 * TILE;         // 2 x 32 KB (dS^T, two 64-query sub-tiles)
  static constexpr int DQ_OFF = DS_OFF + 65536;   // 32 KB fp32 staging (two 32-column sub-tiles)
  static constexpr int LD_OFF = DQ_OFF + 32768;   // [2][256] floats: lse*log2e | delta
  static constexpr int BAR_OFF = LD_OFF + 2048;
  static constexpr int BYTES = BAR_OFF + 256 + 1024;  // + alignment slack
};

__global__ void __launch_bounds__(BWD2_THREADS, 1)
attn_bwd_pp_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                   const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmDO,
                   const __grid_constant__ CUtensorMap tmDQ, const AttnBwdArgs a) {
  constexpr int D = 64;
  using L = AttnBwd2Smem;
  constexpr int TILE = L::TILE;
  constexpr uint32_t TMEM_COLS = 512;
  constexpr uint32_t ST_COL = 0, DPT_COL = 128, DV_COL = 256, DK_COL = 320, DQ_COL = 384;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                              ~uintptr_t(1023));
  uint8_t* sK = smem + L::K_OFF;
  uint8_t* sV = smem + L::V_OFF;
  uint8_t* sQ = smem + L::Q_OFF;
  uint8_t* sDO = smem + L::DO_OFF;
  uint8_t* sDS = smem + L::DS_OFF;
  uint8_t* sDQ = smem + L::DQ_OFF;
  float* sLD = reinterpret_cast<float*>(smem + L::LD_OFF);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::BAR_OFF);
  uint64_t* kv_full = bars + 0;
  uint64_t* qdo_full = bars + 1;   // [2]
  uint64_t* qdo_empty = bars + 3;  // [2]
  uint64_t* sdp_full = bars + 5;
  uint64_t* pds_full = bars + 6;   // 8 compute warps
  uint64_t* dq_full = bars + 7;
  uint64_t* dq_free = bars + 8;    // 4 dQ-writer warps
  uint64_t* acc_full = bars + 9;
  uint64_t* ld_ready = bars + 10;  // [2] lse / delta of a query block staged (256 threads)
  uint64_t* stg_free = bars + 12;  // dQ staging tile reusable
  uint64_t* stg_full = bars + 13;  // dQ staging tile written (128 threads)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 14);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nq = (a.S + 127) / 128;
  const int j = blockIdx.y;  // key block; early key blocks have the most work and go first
  const int bh = blockIdx.x;
  const int b = bh / a.H, h = bh % a.H;
  const int i0 = a.causal ? j : 0;
  const int niter = nq - i0;
  const long long bh_off = ((long long)b * a.H + h) * a.S;

  if (threadIdx.x == 0) {
    mbar_init(kv_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&qdo_full[i], 1);
      mbar_init(&qdo_empty[i], 1);
    }
    mbar_init(sdp_full, 1);
    mbar_init(pds_full, 8);
    mbar_init(dq_full, 1);
    mbar_init(dq_free, 4);
    mbar_init(acc_full, 1);
    mbar_init(&ld_ready[0], 256);
    mbar_init(&ld_ready[1], 256);
    mbar_init(stg_free, 1);
    mbar_init(stg_full, 128);
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 13) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
    tc_fence_before();
  }
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp >= 12) {
    // =================================================================== control
    reg_alloc_dec<40>();
    if (warp == 12 && lane == 0) {
      // ------------------------------------------------------------ TMA producer
      auto load_tile = [&](uint8_t* dst, const CUtensorMap* tm, uint64_t* bar, int row0) {
        tma_load_4d(dst, tm, bar, 0, h, row0, b);
      };
      mbar_expect_tx(kv_full, 2 * TILE);
      load_tile(sK, &tmK, kv_full, j * 128);
      load_tile(sV, &tmV, kv_full, j * 128);
      for (int it = 0; it < niter; ++it) {
        const int st = it & 1;
        if (!mbar_wait(&qdo_empty[st], ((it >> 1) & 1) ^ 1, abort_flag)) {
          att_error(a.status, abort_flag, NKB_ERR_EMPTY_WAIT);
          break;
        }
        mbar_expect_tx(&qdo_full[st], 2 * TILE);
        load_tile(sQ + st * TILE, &tmQ, &qdo_full[st], (i0 + it) * 128);
        load_tile(sDO + st * TILE, &tmDO, &qdo_full[st], (i0 + it) * 128);
      }
    } else if (warp == 13 && lane == 0) {
      // -------------------------------------------------------------- MMA issuer
      constexpr uint32_t idesc_s = umma_idesc_bf16(128, 128, 0, 0);  // S^T, dP^T
      constexpr uint32_t idesc_ts = umma_idesc_bf16(128, D, 0, 1);   // dV, dK: A from TMEM
      constexpr uint32_t idesc_dq = umma_idesc_bf16(128, D, 1, 1);   // dQ: both MN-major
      // descriptors are built once; per MMA only the start-address field (16-byte units) moves
      const uint64_t dK_k = umma_desc_sw128(smem_u32(sK), 16, 1024);      // K, K-major (A of S^T)
      const uint64_t dV_k = umma_desc_sw128(smem_u32(sV), 16, 1024);      // V, K-major (A of dP^T)
      const uint64_t dK_mn = umma_desc_sw128(smem_u32(sK), 16384, 1024);  // K, MN-major (B of dQ)
      const uint64_t dQ_k0 = umma_desc_sw128(smem_u32(sQ), 16, 1024);     // Q, K-major (B of S^T)
      const uint64_t dDO_k0 = umma_desc_sw128(smem_u32(sDO), 16, 1024);
      const uint64_t dQ_mn0 = umma_desc_sw128(smem_u32(sQ), 16384, 1024);   // Q, MN-major (B of dK)
      const uint64_t dDO_mn0 = umma_desc_sw128(smem_u32(sDO), 16384, 1024);
      const uint64_t dDS0 = umma_desc_sw128(smem_u32(sDS), 16384, 1024);    // dS^T, MN-major A
      auto issue_dq = [&](int it) {
        const uint64_t dds = dDS0 + (uint32_t)(it & 1) * (32768 >> 4);
#pragma unroll
        for (int k = 0; k < 8; ++k)  // 16 keys per MMA
          umma_bf16_ss(tmem_base + DQ_COL, dds + k * 128, dK_mn + k * 128, idesc_dq,
                       k > 0 ? 1u : 0u);
        umma_commit(dq_full);
      };
      bool ok = mbar_wait(kv_full, 0, abort_flag);
      if (!ok) att_error(a.status, abort_flag, NKB_ERR_TMA_WAIT);
      for (int it = 0; it < niter && ok; ++it) {
        const int st = it & 1;
        if (!mbar_wait(&qdo_full[st], (it >> 1) & 1, abort_flag)) {
          att_error(a.status, abort_flag, NKB_ERR_TMA_WAIT);
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t soff = (uint32_t)st * (TILE >> 4);
        // S^T = K Q^T ; dP^T = V dO^T   (the tensor pipe runs in order, so the P^T / dS^T
        // of the previous block have been consumed before these overwrite them)
#pragma unroll
        for (int k = 0; k < 4; ++k)
          umma_bf16_ss(tmem_base + ST_COL, dK_k + k * 2, dQ_k0 + soff + k * 2, idesc_s,
                       k > 0 ? 1u : 0u);
#pragma unroll
        for (int k = 0; k < 4; ++k)
          umma_bf16_ss(tmem_base + DPT_COL, dV_k + k * 2, dDO_k0 + soff + k * 2, idesc_s,
                       k > 0 ? 1u : 0u);
        umma_commit(sdp_full);
        if (it > 0) {
          // dQ of the previous block, once the writer has read the one before it
          if (it > 1 && !mbar_wait(dq_free, (it - 2) & 1, abort_flag)) {
            att_error(a.status, abort_flag, NKB_ERR_ACC_FREE);
            ok = false;
            break;
          }
          tc_fence_after();
          issue_dq(it - 1);
        }
        if (!mbar_wait(pds_full, it & 1, abort_flag)) {
          att_error(a.status, abort_flag, NKB_ERR_ACC_WAIT);
          ok = false;
          break;
        }
        tc_fence_after();
        // dV += P^T dO ; dK += dS^T Q   (contraction over the 128 queries; A from TMEM:
        // 16 queries = 8 columns of bf16 pairs, warpgroup w's columns start at 64w)
#pragma unroll
        for (int k = 0; k < 8; ++k)
          umma_bf16_ts(tmem_base + DV_COL, tmem_base + ST_COL + (k >> 2) * 64 + (k & 3) * 8,
                       dDO_mn0 + soff + k * 128, idesc_ts, (it > 0 || k > 0) ? 1u : 0u);
#pragma unroll
        for (int k = 0; k < 8; ++k)
          umma_bf16_ts(tmem_base + DK_COL, tmem_base + DPT_COL + (k >> 2) * 64 + (k & 3) * 8,
                       dQ_mn0 + soff + k * 128, idesc_ts, (it > 0 || k > 0) ? 1u : 0u);
        umma_commit(&qdo_empty[st]);
      }
      if (ok && niter > 0) {
        if (niter > 1 && !mbar_wait(dq_free, (niter - 2) & 1, abort_flag)) {
          att_error(a.status, abort_flag, NKB_ERR_ACC_FREE);
        } else {
          tc_fence_after();
          issue_dq(niter - 1);
          umma_commit(acc_full);
        }
      }
    }
  } else if (warp >= 8) {
    // ================================================================= dQ writer
    reg_alloc_dec<88>();
    const int r = (warp & 3) * 32 + lane;  // query row inside the block (TMEM lane)
    const uint32_t t_lane = tmem_base + (uint32_t((warp & 3) * 32) << 16);
    for (int it = 0; it < niter; ++it) {
      if (!mbar_wait(dq_full, it & 1, abort_flag)) {
        att_error(a.status, abort_flag, NKB_ERR_ACC_WAIT);
        break;
      }
      tc_fence_after();
      uint32_t v[64];
      tmem_ld_32x32(t_lane + DQ_COL, v);
      tmem_ld_32x32(t_lane + DQ_COL + 32, v + 32);
      tmem_ld_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(dq_free);
      // the previous reduce must have finished reading the staging tile
      if (threadIdx.x == 256) {
        tma_store_wait_read<0>();
        mbar_arrive(stg_free);
      }
      if (!mbar_wait(stg_free, it & 1, abort_flag)) {
        att_error(a.status, abort_flag, NKB_ERR_EMPTY_WAIT);
        break;
      }
#pragma unroll
      for (int c = 0; c < 16; ++c) {  // 16-byte chunk c of the row: sub-tile c>>3, chunk c&7
        float4 f = make_float4(__uint_as_float(v[4 * c]) * a.scale, __uint_as_float(v[4 * c + 1]) * a.scale,
                               __uint_as_float(v[4 * c + 2]) * a.scale, __uint_as_float(v[4 * c + 3]) * a.scale);
        *reinterpret_cast<float4*>(sDQ + (c >> 3) * 16384 + sw128_off(r, c & 7)) = f;
      }
      fence_proxy_async_smem();
      mbar_arrive(stg_full);
      if (threadIdx.x == 256) {
        if (!mbar_wait(stg_full, it & 1, abort_flag)) {
          att_error(a.status, abort_flag, NKB_ERR_EMPTY_WAIT);
          break;
        }
        tma_reduce_add_3d(&tmDQ, sDQ, 0, (i0 + it) * 128, bh);
        tma_reduce_add_3d(&tmDQ, sDQ + 16384, 32, (i0 + it) * 128, bh);
        tma_store_commit();
      }
    }
    if (threadIdx.x == 256) tma_store_wait<0>();
  } else {
    // =================================================================== compute
    reg_alloc_inc<184>();
    const int w = warp >> 2;                 // warpgroup: query columns [64w, 64w+64)
    const int r = (warp & 3) * 32 + lane;    // key row inside the block (TMEM lane)
    const int tid = threadIdx.x;             // 0..255
    const uint32_t t_lane = tmem_base + (uint32_t((warp & 3) * 32) << 16);
    // lse * log2(e) (threads 0-127) / delta (threads 128-255) of query (block, tid & 127)
    auto fetch_ld = [&](int it) -> float {
      const int qi = (i0 + it) * 128 + (tid & 127);
      if (qi >= a.S) return tid < 128 ? INFINITY : 0.f;
      return tid < 128 ? a.lse[bh_off + qi] * LOG2E : a.delta[bh_off + qi];
    };
    if (niter > 0) {
      sLD[tid] = fetch_ld(0);
      mbar_arrive(&ld_ready[0]);
    }
    bool ok = true;
    for (int it = 0; it < niter; ++it) {
      const int i = i0 + it;
      float nxt = 0.f;
      if (it + 1 < niter) nxt = fetch_ld(it + 1);
      if (!mbar_wait(&ld_ready[it & 1], (it >> 1) & 1, abort_flag)) {  // lse / delta staged
        att_error(a.status, abort_flag, NKB_ERR_EMPTY_WAIT);
        ok = false;
        break;
      }
      const float* sL = sLD + (it & 1) * 256 + w * 64;
      const float* sDl = sL + 128;
      if (!mbar_wait(sdp_full, it & 1, abort_flag)) {
        att_error(a.status, abort_flag, NKB_ERR_ACC_WAIT);
        ok = false;
        break;
      }
      tc_fence_after();
      uint32_t s[64], dp[64];
      tmem_ld_32x32(t_lane + ST_COL + w * 64, s);
      tmem_ld_32x32(t_lane + ST_COL + w * 64 + 32, s + 32);
      tmem_ld_32x32(t_lane + DPT_COL + w * 64, dp);
      tmem_ld_32x32(t_lane + DPT_COL + w * 64 + 32, dp + 32);
      tmem_ld_wait();
      const bool diag = a.causal && i == j;
      uint32_t pk[32], dk[32];
#pragma unroll
      for (int e = 0; e < 64; e += 4) {
        const float4 l4 = *reinterpret_cast<const float4*>(sL + e);
        const float4 d4 = *reinterpret_cast<const float4*>(sDl + e);
        float p0 = ex2_f32(fmaf(__uint_as_float(s[e]), a.scale_log2, -l4.x));
        float p1 = ex2_f32(fmaf(__uint_as_float(s[e + 1]), a.scale_log2, -l4.y));
        float p2 = ex2_f32(fmaf(__uint_as_float(s[e + 2]), a.scale_log2, -l4.z));
        float p3 = ex2_f32(fmaf(__uint_as_float(s[e + 3]), a.scale_log2, -l4.w));
        if (diag) {  // key r may only see queries >= r
          const int q = w * 64 + e;
          if (r > q) p0 = 0.f;
          if (r > q + 1) p1 = 0.f;
          if (r > q + 2) p2 = 0.f;
          if (r > q + 3) p3 = 0.f;
        }
        const float g0 = p0 * (__uint_as_float(dp[e]) - d4.x);
        const float g1 = p1 * (__uint_as_float(dp[e + 1]) - d4.y);
        const float g2 = p2 * (__uint_as_float(dp[e + 2]) - d4.z);
        const float g3 = p3 * (__uint_as_float(dp[e + 3]) - d4.w);
        pk[e >> 1] = pack_bf16x2(p0, p1);
        pk[(e >> 1) + 1] = pack_bf16x2(p2, p3);
        dk[e >> 1] = pack_bf16x2(g0, g1);
        dk[(e >> 1) + 1] = pack_bf16x2(g2, g3);
      }
      tmem_st_32x16(t_lane + ST_COL + w * 64, pk);
      tmem_st_32x16(t_lane + ST_COL + w * 64 + 16, pk + 16);
      tmem_st_32x16(t_lane + DPT_COL + w * 64, dk);
      tmem_st_32x16(t_lane + DPT_COL + w * 64 + 16, dk + 16);
      uint8_t* ds_tile = sDS + (it & 1) * 32768 + w * 16384;
#pragma unroll
      for (int q = 0; q < 8; ++q)
        *reinterpret_cast<uint4*>(ds_tile + sw128_off(r, q)) =
            make_uint4(dk[4 * q], dk[4 * q + 1], dk[4 * q + 2], dk[4 * q + 3]);
      tmem_st_wait();
      fence_proxy_async_smem();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(pds_full);
      if (it + 1 < niter) {
        sLD[((it + 1) & 1) * 256 + tid] = nxt;
        mbar_arrive(&ld_ready[(it + 1) & 1]);
      }
    }
    if (ok && niter > 0 && mbar_wait(acc_full, 0, abort_flag)) {
      tc_fence_after();
      // dV, dK: warpgroup w stores head-dim columns [32w, 32w+32) of key row r
      const int ki = j * 128 + r;
      const long long off = (long long)b * a.sb + (long long)h * a.sh + (long long)ki * a.ss + w * 32;
#pragma unroll
      for (int which = 0; which < 2; ++which) {
        __nv_bfloat16* dst = (which == 0 ? a.dv : a.dk) + off;
        const float mul = which == 0 ? 1.f : a.scale;
        uint32_t v[32];
        tmem_ld_32x32(t_lane + (which == 0 ? DV_COL : DK_COL) + w * 32, v);
        tmem_ld_wait();
        if (ki < a.S) {
#pragma unroll
          for (int q = 0; q < 4; ++q)
            *reinterpret_cast<uint4*>(dst + q * 8) = make_uint4(
                pack_bf16x2(__uint_as_float(v[8 * q]) * mul, __uint_as_float(v[8 * q + 1]) * mul),
                pack_bf16x2(__uint_as_float(v[8 * q + 2]) * mul, __uint_as_float(v[8 * q + 3]) * mul),
                pack_bf16x2(__uint_as_float(v[8 * q + 4]) * mul, __uint_as_float(v[8 * q + 5]) * mul),
                pack_bf16x2(__uint_as_float(v[8 * q + 6]) * mul, __uint_as_float(v[8 * q + 7]) * mul));
        }
      }
    } else if (ok && niter > 0) {
      att_error(a.status, abort_flag, NKB_ERR_ACC_WAIT);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 13) {
    if (*abort_flag)
      for (int i = 0; i < 1000; ++i) __nanosleep(1000);
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}
