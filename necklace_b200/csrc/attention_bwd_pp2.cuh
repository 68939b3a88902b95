// Variant of the warp-specialised flash-attention backward (attention_bwd_pp.cuh) with one MMA
// issuer per 64-query half (included by attention_sm100.cu inside namespace nkb; selected
// with nkb_attn_set_bwd_impl(2)).  On B200 it measured ~10 % slower than the single-issuer
// form for S = 1024 because S^T / dP^T then take 16 instead of 8 tensor-core instructions
// per block and an instruction of N = 64 costs as much as one of N = 128; it is kept for
// longer sequences and as a reference for the barrier protocol between two issuers.
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
//   warps 13-14 tcgen05.mma issuers, one per compute warpgroup: each 64-query half of a
//               block has its own S^T / dP^T columns, barriers and issuing thread, so the
//               tensor pipe works for one half while the other warpgroup computes (an
//               issuing thread blocks while the pipe is busy; one thread for both halves
//               serialised them).  The second issuer also issues dQ = dS K of the block.
//   warp 15     idle (completes the fourth warpgroup for setmaxnreg).
//
//   TMEM columns: S^T [0,128) (half w at 64w; its P^T over [64w, 64w+32))
//                 dP^T [128,256) (dS^T likewise)  dV [256,320)  dK [320,384)  dQ [384,448)
//
// lse / delta of the query block are staged in shared memory (they index columns here),
// fetched one block ahead.  All waits are bounded.  The reference has no attention layer.
#pragma once

constexpr int BWD3_THREADS = 512;
// setmaxnreg budget: the CTA owns threads x 128 registers (the compile-time cap)
static_assert(256 * 184 + 128 * 88 + 128 * 40 <= BWD3_THREADS * 128, "register budget");

struct AttnBwd3Smem {
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

__global__ void __launch_bounds__(BWD3_THREADS, 1)
attn_bwd_pp2_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                   const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmDO,
                   const __grid_constant__ CUtensorMap tmDQ, const AttnBwdArgs a) {
  constexpr int D = 64;
  using L = AttnBwd3Smem;
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
  uint64_t* sdp_full = bars + 5;   // [2] per half: S^T / dP^T ready
  uint64_t* pds_full = bars + 7;   // [2] per half: P^T / dS^T written (4 compute warps)
  uint64_t* dq_full = bars + 9;
  uint64_t* dq_free = bars + 10;   // 4 dQ-writer warps
  uint64_t* acc_full = bars + 11;  // both issuers
  uint64_t* ld_ready = bars + 12;  // [2] lse / delta of a query block staged (256 threads)
  uint64_t* stg_free = bars + 14;  // dQ staging tile reusable
  uint64_t* stg_full = bars + 15;  // dQ staging tile written (128 threads)
  uint64_t* dq_done = bars + 16;   // [2] dQ MMA of block i retired (index i & 1): its dS^T buffer is free
  uint64_t* ds_ready = bars + 18;  // [2] half 0 of dS^T of block i (index i & 1) is in shared memory
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 20);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nq = (a.S + 127) / 128;
  const int j = blockIdx.y;  // key block; early key blocks have the most work and go first
  const int bh = blockIdx.x;
  const int b = bh / a.H, h = bh % a.H;
  const int i0 = a.causal ? j : 0;
  const int niter = nq - i0;
  const long long bh_off = ((long long)b * a.H + h) * a.S;

  // The TMA thread sets up the barriers and puts the first loads (K, V, two Q / dO stages) in
  // flight before the CTA-wide syncs, so they overlap the TMEM allocation and zero fill.
  if (threadIdx.x == 384) {
    mbar_init(kv_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&qdo_full[i], 1);
      mbar_init(&qdo_empty[i], 2);  // both issuers release a Q / dO stage
      mbar_init(&sdp_full[i], 1);
      mbar_init(&pds_full[i], 4);
      mbar_init(&dq_done[i], 1);
      mbar_init(&ds_ready[i], 4);
    }
    mbar_init(dq_full, 1);
    mbar_init(dq_free, 4);
    mbar_init(acc_full, 2);
    mbar_init(&ld_ready[0], 256);
    mbar_init(&ld_ready[1], 256);
    mbar_init(stg_free, 1);
    mbar_init(stg_full, 128);
    *abort_flag = 0;
    mbar_fence_init();
    mbar_expect_tx(kv_full, 2 * TILE);
    tma_load_4d(sK, &tmK, kv_full, 0, h, j * 128, b);
    tma_load_4d(sV, &tmV, kv_full, 0, h, j * 128, b);
    for (int it = 0; it < 2 && it < niter; ++it) {
      mbar_expect_tx(&qdo_full[it], 2 * TILE);
      tma_load_4d(sQ + it * TILE, &tmQ, &qdo_full[it], 0, h, (i0 + it) * 128, b);
      tma_load_4d(sDO + it * TILE, &tmDO, &qdo_full[it], 0, h, (i0 + it) * 128, b);
    }
  }
  if (warp == 13) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
    tc_fence_before();
  }
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // dV / dK accumulate from two issuing threads whose first MMAs are not ordered against
  // each other, so the accumulators start from explicit zeros and every MMA accumulates
  if (warp < 4) {
    uint32_t z[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) z[i] = 0u;
#pragma unroll
    for (int c = 0; c < 8; ++c)
      tmem_st_32x16(tmem_base + (uint32_t(warp * 32) << 16) + DV_COL + c * 16, z);
    tmem_st_wait();
    tc_fence_before();
  }
  __syncthreads();
  tc_fence_after();

  if (warp >= 12) {
    // =================================================================== control
    reg_alloc_dec<40>();
    if (warp == 12 && lane == 0) {
      // ------------------------------------------------------------ TMA producer
      auto load_tile = [&](uint8_t* dst, const CUtensorMap* tm, uint64_t* bar, int row0) {
        tma_load_4d(dst, tm, bar, 0, h, row0, b);
      };
      for (int it = 2; it < niter; ++it) {  // stages 0 and 1 were filled before the syncs
        const int st = it & 1;
        if (!mbar_wait(&qdo_empty[st], ((it >> 1) & 1) ^ 1, abort_flag)) {
          att_error(a.status, abort_flag, NKB_ERR_EMPTY_WAIT);
          break;
        }
        mbar_expect_tx(&qdo_full[st], 2 * TILE);
        load_tile(sQ + st * TILE, &tmQ, &qdo_full[st], (i0 + it) * 128);
        load_tile(sDO + st * TILE, &tmDO, &qdo_full[st], (i0 + it) * 128);
      }
    } else if ((warp == 13 || warp == 14) && lane == 0) {
      // ------------------------------------- MMA issuer of query half w = warp - 13
      const int w = warp - 13;
      constexpr uint32_t idesc_s = umma_idesc_bf16(128, 64, 0, 0);   // S^T, dP^T halves
      constexpr uint32_t idesc_ts = umma_idesc_bf16(128, D, 0, 1);   // dV, dK: A from TMEM
      constexpr uint32_t idesc_dq = umma_idesc_bf16(128, D, 1, 1);   // dQ: both MN-major
      // descriptors are built once; per MMA only the start-address field (16-byte units)
      // moves.  Half w of a Q / dO tile starts 64 rows = 8192 bytes in.
      const uint32_t hoff = (uint32_t)w * (8192 >> 4);
      const uint64_t dK_k = umma_desc_sw128(smem_u32(sK), 16, 1024);      // K, K-major (A of S^T)
      const uint64_t dV_k = umma_desc_sw128(smem_u32(sV), 16, 1024);      // V, K-major (A of dP^T)
      const uint64_t dK_mn = umma_desc_sw128(smem_u32(sK), 16384, 1024);  // K, MN-major (B of dQ)
      const uint64_t dQ_k0 = umma_desc_sw128(smem_u32(sQ), 16, 1024) + hoff;    // B of S^T
      const uint64_t dDO_k0 = umma_desc_sw128(smem_u32(sDO), 16, 1024) + hoff;  // B of dP^T
      const uint64_t dQ_mn0 = umma_desc_sw128(smem_u32(sQ), 16384, 1024) + hoff;   // B of dK
      const uint64_t dDO_mn0 = umma_desc_sw128(smem_u32(sDO), 16384, 1024) + hoff; // B of dV
      const uint64_t dDS0 = umma_desc_sw128(smem_u32(sDS), 16384, 1024);  // dS^T, MN-major A
      const uint32_t t_st = tmem_base + ST_COL + w * 64, t_dpt = tmem_base + DPT_COL + w * 64;
      bool ok = true;
      auto wait_or_fail = [&](uint64_t* bar, uint32_t parity, int code) {
        if (ok && !mbar_wait(bar, parity, abort_flag)) {
          att_error(a.status, abort_flag, code);
          ok = false;
        }
      };
      wait_or_fail(kv_full, 0, NKB_ERR_TMA_WAIT);
      for (int it = 0; it < niter && ok; ++it) {
        const int st = it & 1;
        wait_or_fail(&qdo_full[st], (it >> 1) & 1, NKB_ERR_TMA_WAIT);
        if (!ok) break;
        tc_fence_after();
        const uint32_t soff = (uint32_t)st * (TILE >> 4);
        // S^T_w = K Q_w^T ; dP^T_w = V dO_w^T.  This thread issued the dV / dK MMAs that read
        // the previous P^T_w / dS^T_w, and its MMAs run in order.
#pragma unroll
        for (int k = 0; k < 4; ++k)
          umma_bf16_ss(t_st, dK_k + k * 2, dQ_k0 + soff + k * 2, idesc_s, k > 0 ? 1u : 0u);
#pragma unroll
        for (int k = 0; k < 4; ++k)
          umma_bf16_ss(t_dpt, dV_k + k * 2, dDO_k0 + soff + k * 2, idesc_s, k > 0 ? 1u : 0u);
        // Warpgroup 0 refills the dS^T buffer of block it-2 once this commit lands; the dQ MMA
        // that reads it belongs to the other issuer, so its retirement is waited for here.
        // (dq_done[b] advances once per two blocks and never runs ahead of this wait.)
        if (w == 0 && it >= 2) wait_or_fail(&dq_done[it & 1], ((it >> 1) - 1) & 1, NKB_ERR_ACC_FREE);
        if (!ok) break;
        umma_commit(&sdp_full[w]);
        wait_or_fail(&pds_full[w], it & 1, NKB_ERR_ACC_WAIT);
        if (!ok) break;
        tc_fence_after();
        // dV += P^T_w dO_w ; dK += dS^T_w Q_w (64 queries: 4 MMAs each, A from TMEM: 16
        // queries = 8 columns of bf16 pairs).  The accumulators were zeroed at start, so both
        // issuers always accumulate and their order does not matter.
#pragma unroll
        for (int k = 0; k < 4; ++k)
          umma_bf16_ts(tmem_base + DV_COL, t_st + k * 8, dDO_mn0 + soff + k * 128, idesc_ts, 1u);
#pragma unroll
        for (int k = 0; k < 4; ++k)
          umma_bf16_ts(tmem_base + DK_COL, t_dpt + k * 8, dQ_mn0 + soff + k * 128, idesc_ts, 1u);
        umma_commit(&qdo_empty[st]);
        if (w == 1) {
          // dQ = dS K of this block: both halves of dS^T are in shared memory and the writer
          // has read the previous dQ.  (Warpgroup 0 may be a block ahead, so its half is
          // signalled on a barrier that alternates with the block index: a parity wait on
          // pds_full[0] could miss a phase.)
          wait_or_fail(&ds_ready[it & 1], (it >> 1) & 1, NKB_ERR_ACC_WAIT);
          if (it > 0) wait_or_fail(dq_free, (it - 1) & 1, NKB_ERR_ACC_FREE);
          if (!ok) break;
          tc_fence_after();
          const uint64_t dds = dDS0 + (uint32_t)(it & 1) * (32768 >> 4);
#pragma unroll
          for (int k = 0; k < 8; ++k)  // 16 keys per MMA
            umma_bf16_ss(tmem_base + DQ_COL, dds + k * 128, dK_mn + k * 128, idesc_dq,
                         k > 0 ? 1u : 0u);
          umma_commit(dq_full);
          umma_commit(&dq_done[it & 1]);
        }
      }
      if (ok && niter > 0) umma_commit(acc_full);
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
      if (!mbar_wait(&sdp_full[w], it & 1, abort_flag)) {
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
      if (lane == 0) {
        mbar_arrive(&pds_full[w]);
        if (w == 0) mbar_arrive(&ds_ready[it & 1]);
      }
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
