// bf16 GEMM for sm_100a: C[M,N] = epilogue(alpha * A[M,K] * B[N,K]^T).
//
// Persistent, warp-specialised kernel, one CTA per SM:
//   warp 0      TMA producer  (cp.async.bulk.tensor, 128-byte swizzle, per-CTA
//               loads only; no cluster multicast)
//   warp 1      tcgen05.mma issuer (one thread), owns the TMEM allocation
//   warps 2..5  epilogue: tcgen05.ld -> registers -> fused math -> global
// The accumulator (128 x BN fp32) lives in TMEM and is double-buffered, so the
// epilogue of tile i overlaps the main loop of tile i+1.
//
// Both operands may be K-major (contraction index contiguous in memory) or
// MN-major (the M / N index contiguous), which covers forward (X W^T), data
// gradient (dY W) and weight gradient (dY^T X) of a linear layer without any
// transpose pass.  This replaces the cuBLAS call under torch's F.linear that the
// reference's tensor-parallel layers use (necklace/frmwrk/pytorch/mpnn/layers.py:239-249,
// :314-328).
//
// All waits are bounded; on a timeout the kernel records a code in
// `status`, releases its TMEM and returns.
#include "ptx.cuh"
#include "nkb_api.h"
#include "comm_dev.cuh"

namespace nkb {

constexpr int BM = 128;
constexpr int BK = 64;  // 64 bf16 = one 128-byte swizzle row
constexpr int UMMA_K = 16;
constexpr int A_STAGE_BYTES = BM * BK * 2;
// warps 0-3: control warpgroup (0 = TMA producer, 1 = MMA issuer / TMEM owner, 2-3 idle);
// warps 4-11: epilogue, two warps per TMEM lane quarter, each taking half of the columns
constexpr int GEMM_THREADS = 384;
constexpr int EPI_WARPS = 8;
// Register hand-over between the warpgroups (setmaxnreg).  The CTA owns what it was launched
// with (threads x the compile-time cap of 168); asking for more would block forever.
constexpr int GEMM_CTRL_REGS = 72, GEMM_EPI_REGS = 216;
static_assert(128 * GEMM_CTRL_REGS + 256 * GEMM_EPI_REGS <= GEMM_THREADS * 168, "register budget");

struct GemmArgs {
  int M, N, K;
  void* C;
  long long ldc;
  int c_fp32;      // 1: C is float, 0: C is bf16
  int accumulate;  // 1: C += result
  float alpha;
  const float* alpha_dev;     // optional device scalar multiplied into alpha
  const __nv_bfloat16* bias;  // [N] or null
  const __nv_bfloat16* res;   // [M, ldres] or null, added after the activation
  long long ldres;
  int epi;                    // NKB_EPI_*
  __nv_bfloat16* aux_out;     // gelu fwd: pre-activation saved here, [M, ldaux]
  const __nv_bfloat16* aux_in;  // gelu bwd: pre-activation read from here
  long long ldaux;
  int num_m_blocks, num_n_blocks;
  int* status;
  // Optional row-block readiness flags (all-gather fused in front of the GEMM):
  // rows [i*rows_per_flag, (i+1)*rows_per_flag) of A may be read once
  // ready_flags[i] >= ready_target.  Null = no waiting.
  const int* ready_flags;
  int rows_per_flag;
  int ready_target;
  // All-gather fused in front of the GEMM (optional, ag_ctas > 0): A is the
  // concatenation of `world` row shards, shard q living at the same offset of rank q's
  // symmetric heap.  The first ag_ctas CTAs pull the remote shards into this rank's
  // copy (plain peer loads) and raise one flag per 128-row block; the GEMM CTAs
  // (which only ever read local memory through TMA) wait on those flags, starting
  // with the local shard.  ready_flags doubles as the flag array; the target epoch is
  // *ag_epoch + 1 (advanced by a follow-up kernel).
  int ag_ctas;
  long long ag_rflag_off;  // byte offset of ready_flags in every member's heap
  CommCtx ag;
  long long ag_data_off;   // byte offset of A inside every heap
  int ag_rows_per_rank;
  long long ag_row_bytes;  // bytes to copy per row (K * 2)
  long long ag_pitch;      // row pitch in bytes
  // Reduce-scatter fused behind the GEMM (optional, rs_on): rows of the result are owned by
  // ranks in contiguous blocks of rs_rows_per_rank.  A partial 128-row tile of another
  // rank's rows is stored straight into the owner's staging slab [src rank][rows_per_rank][N]
  // (peer stores, bf16) followed by a per-tile flag.  Every n-block is walked with the
  // other owners' rows first and this rank's own rows last: by then the peers' partial tiles
  // of those rows have usually arrived, and the epilogue of an own tile waits for their
  // flags, adds them to its fp32 accumulator, applies bias / residual and writes the final
  // [rows_per_rank, N] block.  No CTA is set aside for the reduction.  Staging may be
  // rewritten by a peer only in the next call, after this rank has entered it (one
  // cross-rank barrier at the start, done by an idle warp; pushes wait for its go word,
  // epoch[2]).  C and res are passed as bases shifted by -rank * rows_per_rank rows so that
  // global row numbers index them.
  int rs_on;
  CommCtx rs;
  long long rs_stage_off;  // byte offset of the staging slabs in every heap
  long long rs_tflag_off;  // byte offset of the tile flags [src][row block][n block]
  int rs_rows_per_rank;
  int rs_bn;               // tile width used by the GEMM CTAs
  // Split-K (optional, split_k > 1): the K range is cut into split_k slices that are
  // scheduled as independent work units, so weight-gradient shapes (few output tiles,
  // very long K) still fill the machine.  Slice s stores its raw fp32 partial tile into
  // splitk_ws[s][M][N]; a small follow-up kernel adds the slices and applies alpha /
  // accumulate / output type.
  int split_k;
  float* splitk_ws;
  // Output (and saved pre-activation) tiles leave through TMA stores when their layout
  // allows it (16-byte aligned base and row pitch): box = 64 columns x 32 rows, 128B swizzle.
  int tma_c, tma_aux;
  CUtensorMap tm_c, tm_aux;
};

// Tile t of the persistent walk -> (m-block, n-block).  The plain walk goes down the m-blocks
// of one n-block before the next n-block.  Fused with a collective (m_major) it finishes all
// n-blocks of an m-block first: with the all-gather in front it starts with this rank's own
// rows (shift), so that the CTAs have local work while the peers' rows arrive; with the
// reduce-scatter behind it starts with the next rank's rows and ends with its own, whose
// partial tiles from the peers have arrived by then.
__device__ __forceinline__ void tile_coords(int t, int num_m, int num_n, int shift, bool m_major,
                                            int& mb, int& nb) {
  if (m_major) {
    mb = (t / num_n + shift) % num_m;
    nb = t % num_n;
  } else {
    mb = (t % num_m + shift) % num_m;
    nb = t / num_m;
  }
}

__device__ __forceinline__ void set_error(int* status, volatile int* abort_flag, int code) {
  *abort_flag = 1;
  if (status) atomicCAS(status, 0, code);
}

// Cross-rank barrier done by one warp on flag slot `slot`.  Returns false on timeout.
__device__ __forceinline__ bool warp_barrier(const CommCtx& c, int slot, int value, int lane) {
  bool ok = true;
  __threadfence_system();
  if (lane < c.world) {
    st_release_sys(flag_ptr(c, lane, slot, c.rank), value);
    ok = wait_flag_ge(flag_ptr(c, c.rank, slot, lane), value);
  }
  return __all_sync(0xffffffffu, ok);
}

// Fused reduce-scatter, start of the kernel (one warp of the first GEMM CTA): once every member
// has entered this call, its staging slab may be written; the go word tells this rank's
// epilogue warps.
__device__ __forceinline__ void rs_open_gate(const GemmArgs& g, int epoch, int lane,
                                             volatile int* abort_flag) {
  const bool ok = warp_barrier(g.rs, 0, 2 * epoch - 1, lane);
  if (lane == 0) {
    if (ok) st_release_sys(g.rs.epoch + 2, epoch);
    else set_error(g.status, abort_flag, NKB_ERR_FLAG_WAIT);
  }
}
// An epilogue warp before its first peer store of the call.
__device__ __forceinline__ bool rs_wait_gate(const GemmArgs& g, int epoch, int lane) {
  bool ok = true;
  if (lane == 0) ok = wait_flag_ge(g.rs.epoch + 2, epoch);
  return __all_sync(0xffffffffu, ok);
}
// An epilogue warp before the epilogue of one of this rank's own tiles: the partial tiles of
// all other members for (row block lb, n-block nb) are in the staging slab.
__device__ __forceinline__ bool rs_wait_partials(const GemmArgs& g, int lb, int nb, int nbk,
                                                 int epoch, int lane) {
  bool ok = true;
  if (lane < g.rs.world && lane != g.rs.rank) {
    const int* tflags = reinterpret_cast<const int*>(
        static_cast<const char*>(g.rs.heap[g.rs.rank]) + g.rs_tflag_off);
    ok = wait_flag_ge(tflags + ((long long)lane * (g.rs_rows_per_rank / 128) + lb) * nbk + nb,
                      epoch);
  }
  return __all_sync(0xffffffffu, ok);
}

// Staging row pointer and flag of the 128-row block that starts at global row `row_blk0`
// for n-block nb (fused reduce-scatter): returns the staging address of (row_blk0 +
// lane_grp*32, n0) in the owner's heap.
__device__ __forceinline__ __nv_bfloat16* rs_tile_dst(const GemmArgs& g, int row_blk0,
                                                      int lane_grp, int n0, int** flag, int nb,
                                                      int nbk) {
  const int R = g.rs_rows_per_rank;
  const int q = row_blk0 / R, lb = (row_blk0 - q * R) / 128;
  char* base = static_cast<char*>(g.rs.heap[q]);
  *flag = reinterpret_cast<int*>(base + g.rs_tflag_off) +
          ((long long)g.rs.rank * (R / 128) + lb) * nbk + nb;
  return reinterpret_cast<__nv_bfloat16*>(base + g.rs_stage_off) +
         ((long long)g.rs.rank * R + lb * 128 + lane_grp * 32) * g.N + n0;
}

// Copy role of the fused all-gather (see GemmArgs).  One flag per 128-row block.
// The copy is a push: a CTA reads a 128-row block of this rank's own shard and stores it
// into one peer's gather buffer (posted writes pipeline over NVLink; peer loads, which are
// ordered system-scope reads, ran one round trip at a time), fences, and raises the block's
// flag in that peer's flag array.  A peer's buffer may be written once that peer has entered
// the kernel (first barrier): everything it launched before, readers of the buffer's previous
// content included, has finished by then.  No barrier is needed at the end: nobody reads
// this rank's memory, and this rank's own stores are fenced before the flags they precede.
__device__ __noinline__ static void ag_copy_role(const GemmArgs& g) {
  const CommCtx& c = g.ag;
  const int e = *reinterpret_cast<volatile int*>(c.epoch) + 1;
  int* flags = const_cast<int*>(g.ready_flags);
  const int R = g.ag_rows_per_rank;
  const int blocks_per_rank = (R + 127) / 128;
  bool ok = cta_barrier(c, 2 * e - 1);  // every rank is in the kernel
  if (!ok) return;
  // local shard: ready at once
  for (int b = blockIdx.x * blockDim.x + threadIdx.x; b < blocks_per_rank;
       b += g.ag_ctas * blockDim.x)
    st_release_sys(flags + c.rank * blocks_per_rank + b, e);
  const char* mine = static_cast<const char*>(c.heap[c.rank]) + g.ag_data_off;
  const int v_per_row = (int)(g.ag_row_bytes >> 4);  // 128 rows of it fit an int by far
  constexpr int AG_UNROLL = 8;
  // (peer, block) units dealt round-robin to the copy CTAs.  A peer's GEMM walks the row
  // blocks starting with its own shard and going up the ranks, so it needs this rank's rows
  // the sooner the closer it sits below this rank: peers are served in that order.
  const int units = (c.world - 1) * blocks_per_rank;
  for (int u = blockIdx.x; u < units; u += g.ag_ctas) {
    const int q = (c.rank + c.world - 1 - u / blocks_per_rank) % c.world;
    const int b = u % blocks_per_rank;
    const long long blk_off = (long long)(c.rank * R + b * 128) * g.ag_pitch;
    const char* src = mine + blk_off;
    char* dst = static_cast<char*>(c.heap[q]) + g.ag_data_off + blk_off;
    const int nrows = min(128, R - b * 128);
    const int total = nrows * v_per_row;
    for (int i0 = threadIdx.x; i0 < total; i0 += (int)blockDim.x * AG_UNROLL) {
      uint4 v[AG_UNROLL];
      long long off[AG_UNROLL];
#pragma unroll
      for (int k = 0; k < AG_UNROLL; ++k) {
        const int i = i0 + k * (int)blockDim.x;
        off[k] = (long long)(i / v_per_row) * g.ag_pitch + ((i % v_per_row) << 4);
        if (i < total) v[k] = *reinterpret_cast<const uint4*>(src + off[k]);
      }
#pragma unroll
      for (int k = 0; k < AG_UNROLL; ++k)
        if (i0 + k * (int)blockDim.x < total) *reinterpret_cast<uint4*>(dst + off[k]) = v[k];
    }
    __threadfence_system();  // this thread's stores have reached the peer
    __syncthreads();
    if (threadIdx.x == 0)
      st_release_sys(reinterpret_cast<int*>(static_cast<char*>(c.heap[q]) + g.ag_rflag_off) +
                         c.rank * blocks_per_rank + b,
                     e);
  }
}

__global__ void epoch_bump_kernel(int* epoch) { epoch[0] += 1; }

// out = (accumulate ? out : 0) + alpha * sum_s ws[s]; 4 elements per thread-iteration
// (N % 4 == 0 and 16-byte aligned rows are guaranteed by the caller).
__global__ void __launch_bounds__(256)
splitk_reduce_kernel(const float* __restrict__ ws, int S, long long MN, int N, void* out,
                     long long ldc, int c_fp32, int accumulate, float alpha,
                     const float* __restrict__ alpha_dev) {
  if (alpha_dev) alpha *= *alpha_dev;
  const long long n4 = MN >> 2;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n4;
       i += (long long)gridDim.x * blockDim.x) {
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int s = 0; s < S; ++s) {
      float4 v = reinterpret_cast<const float4*>(ws + (long long)s * MN)[i];
      acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
    }
    const long long e = i << 2, row = e / N, col = e % N;
    acc.x *= alpha; acc.y *= alpha; acc.z *= alpha; acc.w *= alpha;
    if (c_fp32) {
      float4* o = reinterpret_cast<float4*>(static_cast<float*>(out) + row * ldc + col);
      if (accumulate) { float4 p = *o; acc.x += p.x; acc.y += p.y; acc.z += p.z; acc.w += p.w; }
      *o = acc;
    } else {
      uint2* o = reinterpret_cast<uint2*>(static_cast<__nv_bfloat16*>(out) + row * ldc + col);
      if (accumulate) {
        uint2 p = *o;
        float2 a = unpack_bf16x2(p.x), b = unpack_bf16x2(p.y);
        acc.x += a.x; acc.y += a.y; acc.z += b.x; acc.w += b.y;
      }
      *o = make_uint2(pack_bf16x2(acc.x, acc.y), pack_bf16x2(acc.z, acc.w));
    }
  }
}

__device__ __forceinline__ float gelu_tanh(float x) {
  const float k0 = 0.7978845608028654f, k1 = 0.044715f;
  float u = k0 * (x + k1 * x * x * x);
  float t;
  asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(u));
  return 0.5f * x * (1.f + t);
}
__device__ __forceinline__ float gelu_tanh_grad(float x) {
  const float k0 = 0.7978845608028654f, k1 = 0.044715f;
  float x2 = x * x;
  float u = k0 * (x + k1 * x * x2);
  float t;
  asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(u));
  float du = k0 * (1.f + 3.f * k1 * x2);
  return 0.5f * (1.f + t) + 0.5f * x * (1.f - t * t) * du;
}

// ---- epilogue staging tile: 32 rows x 128 bytes per warp, 16-byte chunks XOR-swizzled
// by (row & 7) so both the row-per-thread and the 4-rows-per-instruction access
// patterns are free of bank conflicts.
constexpr int EPI_STAGE_BYTES = 32 * 128;

__device__ __forceinline__ uint4 stage_get(const uint8_t* stg, int row, int chunk) {
  return *reinterpret_cast<const uint4*>(stg + row * 128 + ((chunk ^ (row & 7)) << 4));
}
__device__ __forceinline__ void stage_set(uint8_t* stg, int row, int chunk, uint4 v) {
  *reinterpret_cast<uint4*>(stg + row * 128 + ((chunk ^ (row & 7)) << 4)) = v;
}
// thread `lane` writes its 64 values as bf16 into row `lane`
__device__ __forceinline__ void stage_put_bf16(uint8_t* stg, int lane, const float* v) {
  __syncwarp();
#pragma unroll
  for (int q = 0; q < 8; ++q)
    stage_set(stg, lane, q,
              make_uint4(pack_bf16x2(v[q * 8 + 0], v[q * 8 + 1]), pack_bf16x2(v[q * 8 + 2], v[q * 8 + 3]),
                         pack_bf16x2(v[q * 8 + 4], v[q * 8 + 5]), pack_bf16x2(v[q * 8 + 6], v[q * 8 + 7])));
}
// Cooperative copies between the staging tile and a [rows_valid x cols_valid]
// global tile (row pitch ld elements).  ESZ = element size; a row of the tile is
// 128 bytes = 8 chunks of CH = 16/ESZ elements.  Instruction i moves rows
// 4i..4i+3, one 16-byte chunk per lane.
template <typename T>
__device__ __forceinline__ void stage_store_t(const uint8_t* stg, int lane, T* gptr, long long ld,
                                              int rows_valid, int cols_valid) {
  constexpr int CH = 16 / (int)sizeof(T);
  const bool vec = ((ld * (long long)sizeof(T)) & 15) == 0 &&
                   (reinterpret_cast<uintptr_t>(gptr) & 15) == 0;
  __syncwarp();
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int row = i * 4 + (lane >> 3), ch = lane & 7;
    if (row < rows_valid && ch * CH < cols_valid) {
      const uint4 v = stage_get(stg, row, ch);
      T* dst = gptr + (long long)row * ld + ch * CH;
      if (vec && (ch + 1) * CH <= cols_valid) {
        *reinterpret_cast<uint4*>(dst) = v;
      } else {
        const T* e = reinterpret_cast<const T*>(&v);
        for (int k = 0; k < CH && ch * CH + k < cols_valid; ++k) dst[k] = e[k];
      }
    }
  }
  __syncwarp();
}
template <typename T>
__device__ __forceinline__ void stage_load_t(uint8_t* stg, int lane, const T* gptr, long long ld,
                                             int rows_valid, int cols_valid) {
  constexpr int CH = 16 / (int)sizeof(T);
  const bool vec = ((ld * (long long)sizeof(T)) & 15) == 0 &&
                   (reinterpret_cast<uintptr_t>(gptr) & 15) == 0;
  __syncwarp();
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int row = i * 4 + (lane >> 3), ch = lane & 7;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (row < rows_valid && ch * CH < cols_valid) {
      const T* src = gptr + (long long)row * ld + ch * CH;
      if (vec && (ch + 1) * CH <= cols_valid) {
        v = *reinterpret_cast<const uint4*>(src);
      } else {
        T* e = reinterpret_cast<T*>(&v);
        for (int k = 0; k < CH && ch * CH + k < cols_valid; ++k) e[k] = src[k];
      }
    }
    stage_set(stg, row, ch, v);
  }
  __syncwarp();
}
__device__ __forceinline__ void stage_store_bf16(const uint8_t* stg, int lane, __nv_bfloat16* g,
                                                 long long ld, int rv, int cv) {
  stage_store_t<__nv_bfloat16>(stg, lane, g, ld, rv, cv);
}
__device__ __forceinline__ void stage_load_bf16(uint8_t* stg, int lane, const __nv_bfloat16* g,
                                                long long ld, int rv, int cv) {
  stage_load_t<__nv_bfloat16>(stg, lane, g, ld, rv, cv);
}
__device__ __forceinline__ void stage_store_f32(const uint8_t* stg, int lane, float* g,
                                                long long ld, int rv, int cv) {
  stage_store_t<float>(stg, lane, g, ld, rv, cv);
}
__device__ __forceinline__ void stage_load_f32(uint8_t* stg, int lane, const float* g, long long ld,
                                               int rv, int cv) {
  stage_load_t<float>(stg, lane, g, ld, rv, cv);
}

// Epilogue of one 128 x BN accumulator slab: this warp's 32 rows (TMEM lanes), BN
// columns starting at global column n0; fused math, then staged coalesced stores.
// Residual / saved-activation rows that the epilogue adds or multiplies do not depend on the
// accumulator: their 32 x 64 bf16 block is copied global -> staging tile with cp.async
// (no registers), for a tile's first chunk before the wait on the accumulator.  Returns
// false (nothing issued) for ragged or unaligned blocks, which take the synchronous load.
__device__ __forceinline__ bool epi_stage_async(uint8_t* stg, int lane, const __nv_bfloat16* src,
                                                long long ld, int row0, int rows_valid, int col0,
                                                int N) {
  const bool ok = src != nullptr && ((ld & 7) == 0) &&
                  ((reinterpret_cast<uintptr_t>(src) & 15) == 0) && rows_valid == 32 &&
                  col0 + 64 <= N;
  if (!ok) return false;
  if (lane == 0) tma_store_wait_read<0>();  // an earlier TMA store may still read the tile
  __syncwarp();
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int row = i * 4 + (lane >> 3), ch = lane & 7;
    const uint32_t dst = smem_u32(stg + row * 128 + ((ch ^ (row & 7)) << 4));
    const __nv_bfloat16* gp = src + (long long)(row0 + row) * ld + col0 + ch * 8;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(gp) : "memory");
  }
  asm volatile("cp.async.commit_group;" ::: "memory");
  return true;
}
__device__ __forceinline__ void epi_stage_async_wait() {
  asm volatile("cp.async.wait_group 0;" ::: "memory");
  __syncwarp();
}

// ---- bf16-output fast path of the epilogue -------------------------------------------
// Straight-line code that runs once per tile is bound by instruction fetch (a trace showed
// ~20 cycles per instruction in the fully unrolled form), so the fast path is ONE copy of a
// 32-column half body inside loops that are not unrolled: chunks of the warp's share, halves
// of a chunk.  Math runs on packed fp32 pairs.  At most one staged input tile (residual,
// saved pre-activation or the old C for accumulation) and no input together with the GELU
// forward (whose first pass uses the staging tile); other combinations take the general form.
// values travel as packed fp32 pairs (one instruction per two columns)
__device__ __forceinline__ void epi_load_half(uint32_t taddr, float alpha, f32x2_t* v) {
  uint32_t r[32];
  tmem_ld_32x32(taddr, r);
  tmem_ld_wait();
  const f32x2_t a2 = f2_pack(alpha, alpha);
#pragma unroll
  for (int i = 0; i < 16; ++i)
    v[i] = f2_mul(f2_pack(__uint_as_float(r[2 * i]), __uint_as_float(r[2 * i + 1])), a2);
}
__device__ __forceinline__ void epi_bias_half(const GemmArgs& g, f32x2_t* v, int c0, int cv,
                                              bool vec) {
  if (!g.bias) return;
  if (vec) {
    const uint4* bp = reinterpret_cast<const uint4*>(g.bias + c0);
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const uint4 b = __ldg(bp + q);
      const uint32_t w[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) v[q * 4 + j] = f2_add(v[q * 4 + j], f2_from_bf16x2(w[j]));
    }
  } else {
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const float b0 = (2 * i < cv) ? __bfloat162float(g.bias[c0 + 2 * i]) : 0.f;
      const float b1 = (2 * i + 1 < cv) ? __bfloat162float(g.bias[c0 + 2 * i + 1]) : 0.f;
      v[i] = f2_add(v[i], f2_pack(b0, b1));
    }
  }
}
// tanh-form GELU and its derivative on packed pairs
__device__ __forceinline__ f32x2_t gelu_tanh2(f32x2_t x) {
  const float k0 = 0.7978845608028654f, k1 = 0.044715f;
  const f32x2_t x2 = f2_mul(x, x);
  const f32x2_t u = f2_mul(x, f2_fma(x2, f2_pack(k0 * k1, k0 * k1), f2_pack(k0, k0)));
  const f32x2_t t = f2_tanh(u);
  const f32x2_t hx = f2_mul(x, f2_pack(0.5f, 0.5f));
  return f2_fma(hx, t, hx);
}
__device__ __forceinline__ f32x2_t gelu_tanh_grad2(f32x2_t x) {
  const float k0 = 0.7978845608028654f, k1 = 0.044715f;
  const f32x2_t x2 = f2_mul(x, x);
  const f32x2_t u = f2_mul(x, f2_fma(x2, f2_pack(k0 * k1, k0 * k1), f2_pack(k0, k0)));
  const f32x2_t t = f2_tanh(u);
  const f32x2_t du = f2_fma(x2, f2_pack(3.f * k0 * k1, 3.f * k0 * k1), f2_pack(k0, k0));
  const f32x2_t one_m_t2 = f2_fma(f2_mul(t, f2_pack(-1.f, -1.f)), t, f2_pack(1.f, 1.f));
  const f32x2_t w = f2_mul(f2_mul(f2_mul(x, f2_pack(0.5f, 0.5f)), one_m_t2), du);
  return f2_add(f2_fma(t, f2_pack(0.5f, 0.5f), f2_pack(0.5f, 0.5f)), w);
}
// thread `lane` writes 16 packed pairs as bf16 into half h of row `lane`
__device__ __forceinline__ void stage_put_half(uint8_t* stg, int lane, int h, const f32x2_t* v) {
#pragma unroll
  for (int q = 0; q < 4; ++q)
    stage_set(stg, lane, 4 * h + q,
              make_uint4(f2_to_bf16x2(v[q * 4 + 0]), f2_to_bf16x2(v[q * 4 + 1]),
                         f2_to_bf16x2(v[q * 4 + 2]), f2_to_bf16x2(v[q * 4 + 3])));
}
// The staging tile goes to global memory: one TMA store issued by lane 0 (the tensor map clips
// rows / columns outside the matrix), else the cooperative copy.  Shared memory is the scarce
// resource here: the MMA operand reads and the TMA operand writes already use most of its
// bandwidth, and a copy by the warp costs a ld.shared + st.global per 512 bytes.
__device__ __forceinline__ void stage_out(const uint8_t* stg, int lane, const CUtensorMap* tm,
                                          bool use_tma, __nv_bfloat16* gptr, long long ld, int row0,
                                          int col0, int rows_valid, int cols_valid) {
  if (use_tma) {
    fence_proxy_async_smem();
    __syncwarp();
    if (lane == 0) {
      tma_store_2d(tm, stg, col0, row0);
      tma_store_commit();
    }
  } else {
    stage_store_bf16(stg, lane, gptr, ld, rows_valid, cols_valid);
  }
}
// before the tile is written again: the store has finished reading it
__device__ __forceinline__ void stage_out_drain(int lane, bool use_tma) {
  if (use_tma) {
    if (lane == 0) tma_store_wait_read<0>();
    __syncwarp();
  }
}

__device__ __forceinline__ void epilogue_chunk_fast(const GemmArgs& g, uint8_t* stg, int lane,
                                                    uint32_t t_c, int row0, int rows_valid,
                                                    int col0, float alpha, bool bias_vec,
                                                    bool in_async) {
  const int cols_valid = (g.N - col0) < 64 ? (g.N - col0) : 64;
  const bool vec_bias = bias_vec && cols_valid == 64 && (col0 & 7) == 0;
  const bool in_res = g.res != nullptr, in_aux = g.epi == NKB_EPI_GELU_BWD;
  const bool in_acc = g.accumulate != 0;
  if (!in_async) stage_out_drain(lane, true);  // the previous chunk's store has read the tile
  if (g.epi == NKB_EPI_GELU_FWD) {
    // first pass: the pre-activation goes out for the backward pass
    __syncwarp();
#pragma unroll 1
    for (int h = 0; h < 2; ++h) {
      f32x2_t v[16];
      epi_load_half(t_c + h * 32, alpha, v);
      epi_bias_half(g, v, col0 + h * 32, cols_valid - h * 32, vec_bias);
      stage_put_half(stg, lane, h, v);
    }
    stage_out(stg, lane, &g.tm_aux, g.tma_aux != 0, g.aux_out + (long long)row0 * g.ldaux + col0,
              g.ldaux, row0, col0, rows_valid, cols_valid);
    stage_out_drain(lane, g.tma_aux != 0);
  } else if (in_async) {
    epi_stage_async_wait();
  } else if (in_res) {
    stage_load_bf16(stg, lane, g.res + (long long)row0 * g.ldres + col0, g.ldres, rows_valid,
                    cols_valid);
  } else if (in_aux) {
    stage_load_bf16(stg, lane, g.aux_in + (long long)row0 * g.ldaux + col0, g.ldaux, rows_valid,
                    cols_valid);
  } else if (in_acc) {
    stage_load_bf16(stg, lane, reinterpret_cast<const __nv_bfloat16*>(g.C) +
                                   (long long)row0 * g.ldc + col0, g.ldc, rows_valid, cols_valid);
  } else {
    __syncwarp();  // the previous chunk's cooperative store has read the tile
  }
#pragma unroll 1
  for (int h = 0; h < 2; ++h) {
    f32x2_t v[16];
    epi_load_half(t_c + h * 32, alpha, v);
    epi_bias_half(g, v, col0 + h * 32, cols_valid - h * 32, vec_bias);
    if (g.epi == NKB_EPI_GELU_FWD) {
#pragma unroll
      for (int i = 0; i < 16; ++i) v[i] = gelu_tanh2(v[i]);
    } else if (g.epi == NKB_EPI_RELU) {
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        float a, b;
        f2_unpack(v[i], a, b);
        v[i] = f2_pack(fmaxf(a, 0.f), fmaxf(b, 0.f));
      }
    }
    if (in_res || in_aux || in_acc) {
      // this thread's own row of the staged input; half h is overwritten right after
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const uint4 z = stage_get(stg, lane, 4 * h + q);
        const uint32_t w[4] = {z.x, z.y, z.z, z.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const f32x2_t f = f2_from_bf16x2(w[j]);
          if (in_aux) v[q * 4 + j] = f2_mul(v[q * 4 + j], gelu_tanh_grad2(f));
          else v[q * 4 + j] = f2_add(v[q * 4 + j], f);
        }
      }
    }
    stage_put_half(stg, lane, h, v);
  }
  stage_out(stg, lane, &g.tm_c, g.tma_c != 0,
            reinterpret_cast<__nv_bfloat16*>(g.C) + (long long)row0 * g.ldc + col0, g.ldc, row0, col0,
            rows_valid, cols_valid);
}

__device__ __forceinline__ bool epi_fast_ok(const GemmArgs& g) {
  const int n_in = (g.res ? 1 : 0) + (g.epi == NKB_EPI_GELU_BWD ? 1 : 0) + (g.accumulate ? 1 : 0);
  return !g.c_fp32 && n_in <= 1 && !(n_in == 1 && g.epi == NKB_EPI_GELU_FWD);
}
// source of the staged input that may be fetched ahead (residual or saved pre-activation)
__device__ __forceinline__ const __nv_bfloat16* epi_async_src(const GemmArgs& g, long long* ld) {
  if (g.res) { *ld = g.ldres; return g.res; }
  if (g.epi == NKB_EPI_GELU_BWD) { *ld = g.ldaux; return g.aux_in; }
  *ld = 0;
  return nullptr;
}
// The warp's share of a tile: chunks [cc0, cc0 + ncw); first_async: the first chunk's input
// is already on its way into the staging tile.
__device__ __forceinline__ void epilogue_fast_tile(const GemmArgs& g, uint8_t* stg, int lane,
                                                   uint32_t t_addr, int row0, int rows_valid,
                                                   int n0, float alpha, bool bias_vec, int cc0,
                                                   int ncw, bool first_async) {
  if (rows_valid == 0) return;
  long long in_ld;
  const __nv_bfloat16* in_src = epi_async_src(g, &in_ld);
#pragma unroll 1
  for (int c = 0; c < ncw; ++c) {
    const int col0 = n0 + (cc0 + c) * 64;
    if (col0 >= g.N) break;  // warp-uniform
    bool in_async = first_async;
    if (c > 0) in_async = epi_stage_async(stg, lane, in_src, in_ld, row0, rows_valid, col0, g.N);
    epilogue_chunk_fast(g, stg, lane, t_addr + (cc0 + c) * 64, row0, rows_valid, col0, alpha,
                        bias_vec, in_async);
  }
}

// MODE 0: plain epilogue; 1: kernel fused with a collective (rs_dst set: raw partial
// sums to the owner's staging slab); 2: split-K (raw fp32 partial sums to raw_dst).
// General form: one 64-column chunk (index cc) of this warp's 32-row slab, fully unrolled.
template <int MODE>
__device__ __forceinline__ void epilogue_chunk_general(const GemmArgs& g, uint8_t* stg, int lane,
                                               uint32_t t_addr, int row0, int rows_valid, int n0,
                                               float alpha, bool bias_vec, int cc,
                                               __nv_bfloat16* rs_dst, long long rs_ld,
                                               float* raw_dst,
                                               const __nv_bfloat16* rs_own = nullptr) {
    uint32_t r[64];
    tmem_ld_32x32(t_addr + cc * 64, r);
    tmem_ld_32x32(t_addr + cc * 64 + 32, r + 32);
    tmem_ld_wait();
    const int col0 = n0 + cc * 64;
    if (rows_valid == 0 || col0 >= g.N) return;  // warp-uniform
    const int cols_valid = (g.N - col0) < 64 ? (g.N - col0) : 64;
    float v[64];
#pragma unroll
    for (int i = 0; i < 64; ++i) v[i] = __uint_as_float(r[i]) * alpha;
    if constexpr (MODE == 2) {
      // split-K: raw fp32 partial sums into this slice's workspace slab (pitch N)
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        const int cv = cols_valid - half * 32;
        if (cv > 0) {
          __syncwarp();
#pragma unroll
          for (int q = 0; q < 8; ++q)
            stage_set(stg, lane, q,
                      make_uint4(r[half * 32 + q * 4], r[half * 32 + q * 4 + 1],
                                 r[half * 32 + q * 4 + 2], r[half * 32 + q * 4 + 3]));
          stage_store_f32(stg, lane, raw_dst + cc * 64 + half * 32, g.N, rows_valid, cv);
        }
      }
      return;
    }
    if constexpr (MODE == 1) {
      if (rs_dst) {
        // fused reduce-scatter: the raw partial sums go to the owner's staging slab;
        // bias / residual are applied by the owner after the cross-rank sum
        stage_put_bf16(stg, lane, v);
        stage_store_bf16(stg, lane, rs_dst + cc * 64, rs_ld, rows_valid, cols_valid);
        return;
      }
      if (rs_own) {
        // own rows: add the other members' partial sums (this lane's row of each slab, read
        // from L2, where the peers' stores arrived); bias, residual and the store follow
        if (lane < rows_valid) {
          const long long slab = (long long)g.rs_rows_per_rank * g.N;
          for (int src = 0; src < g.rs.world; ++src) {
            if (src == g.rs.rank) continue;
            const __nv_bfloat16* prow = rs_own + src * slab + (long long)lane * g.N + cc * 64;
#pragma unroll
            for (int h = 0; h < 2; ++h) {
              uint4 pv[4];
#pragma unroll
              for (int q = 0; q < 4; ++q)
                if ((h * 4 + q) * 8 < cols_valid) pv[q] = ld_cg_v4(prow + (h * 4 + q) * 8);
#pragma unroll
              for (int q = 0; q < 4; ++q) {
                if ((h * 4 + q) * 8 >= cols_valid) continue;
                const uint32_t w[4] = {pv[q].x, pv[q].y, pv[q].z, pv[q].w};
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                  const float2 f = unpack_bf16x2(w[j]);
                  v[(h * 4 + q) * 8 + 2 * j] += f.x;
                  v[(h * 4 + q) * 8 + 2 * j + 1] += f.y;
                }
              }
            }
          }
        }
      }
    }
    if (g.bias) {
      if (bias_vec && cols_valid == 64 && (col0 & 7) == 0) {
        const uint4* bp = reinterpret_cast<const uint4*>(g.bias + col0);
#pragma unroll
        for (int q = 0; q < 8; ++q) {
          uint4 b = __ldg(bp + q);
          uint32_t w[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            float2 f = unpack_bf16x2(w[j]);
            v[q * 8 + 2 * j] += f.x;
            v[q * 8 + 2 * j + 1] += f.y;
          }
        }
      } else {
#pragma unroll
        for (int i = 0; i < 64; ++i)
          if (i < cols_valid) v[i] += __bfloat162float(g.bias[col0 + i]);
      }
    }
    if (g.epi == NKB_EPI_GELU_FWD) {
      stage_put_bf16(stg, lane, v);
      stage_store_bf16(stg, lane, g.aux_out + (long long)row0 * g.ldaux + col0, g.ldaux,
                       rows_valid, cols_valid);
#pragma unroll
      for (int i = 0; i < 64; ++i) v[i] = gelu_tanh(v[i]);
    } else if (g.epi == NKB_EPI_GELU_BWD) {
      stage_load_bf16(stg, lane, g.aux_in + (long long)row0 * g.ldaux + col0, g.ldaux,
                      rows_valid, cols_valid);
#pragma unroll
      for (int q = 0; q < 8; ++q) {
        uint4 z = stage_get(stg, lane, q);
        uint32_t w[4] = {z.x, z.y, z.z, z.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          float2 f = unpack_bf16x2(w[j]);
          v[q * 8 + 2 * j] *= gelu_tanh_grad(f.x);
          v[q * 8 + 2 * j + 1] *= gelu_tanh_grad(f.y);
        }
      }
    } else if (g.epi == NKB_EPI_RELU) {
#pragma unroll
      for (int i = 0; i < 64; ++i) v[i] = fmaxf(v[i], 0.f);
    }
    if (g.res) {
      stage_load_bf16(stg, lane, g.res + (long long)row0 * g.ldres + col0, g.ldres, rows_valid,
                      cols_valid);
#pragma unroll
      for (int q = 0; q < 8; ++q) {
        uint4 z = stage_get(stg, lane, q);
        uint32_t w[4] = {z.x, z.y, z.z, z.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          float2 f = unpack_bf16x2(w[j]);
          v[q * 8 + 2 * j] += f.x;
          v[q * 8 + 2 * j + 1] += f.y;
        }
      }
    }
    if (g.c_fp32) {
      float* cbase = reinterpret_cast<float*>(g.C) + (long long)row0 * g.ldc + col0;
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        const int cv = cols_valid - half * 32;
        if (cv > 0) {
        if (g.accumulate) {
          stage_load_f32(stg, lane, cbase + half * 32, g.ldc, rows_valid, cv);
#pragma unroll
          for (int q = 0; q < 8; ++q) {
            uint4 z = stage_get(stg, lane, q);
            v[half * 32 + q * 4 + 0] += __uint_as_float(z.x);
            v[half * 32 + q * 4 + 1] += __uint_as_float(z.y);
            v[half * 32 + q * 4 + 2] += __uint_as_float(z.z);
            v[half * 32 + q * 4 + 3] += __uint_as_float(z.w);
          }
        }
        __syncwarp();
#pragma unroll
        for (int q = 0; q < 8; ++q)
          stage_set(stg, lane, q,
                    make_uint4(__float_as_uint(v[half * 32 + q * 4]),
                               __float_as_uint(v[half * 32 + q * 4 + 1]),
                               __float_as_uint(v[half * 32 + q * 4 + 2]),
                               __float_as_uint(v[half * 32 + q * 4 + 3])));
        stage_store_f32(stg, lane, cbase + half * 32, g.ldc, rows_valid, cv);
        }
      }
    } else {
      __nv_bfloat16* cbase =
          reinterpret_cast<__nv_bfloat16*>(g.C) + (long long)row0 * g.ldc + col0;
      if (g.accumulate) {
        stage_load_bf16(stg, lane, cbase, g.ldc, rows_valid, cols_valid);
#pragma unroll
        for (int q = 0; q < 8; ++q) {
          uint4 z = stage_get(stg, lane, q);
          uint32_t w[4] = {z.x, z.y, z.z, z.w};
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            float2 f = unpack_bf16x2(w[j]);
            v[q * 8 + 2 * j] += f.x;
            v[q * 8 + 2 * j + 1] += f.y;
          }
        }
      }
      stage_put_bf16(stg, lane, v);
      stage_store_bf16(stg, lane, cbase, g.ldc, rows_valid, cols_valid);
    }
}

// The warp handles chunks [cc0, cc0 + NCW) of the slab (general form).
template <int BN, int MODE, int NCW>
__device__ __forceinline__ void epilogue_tile(const GemmArgs& g, uint8_t* stg, int lane,
                                              uint32_t t_addr, int row0, int rows_valid, int n0,
                                              float alpha, bool bias_vec, int cc0,
                                              __nv_bfloat16* rs_dst = nullptr,
                                              long long rs_ld = 0, float* raw_dst = nullptr,
                                              const __nv_bfloat16* rs_own = nullptr) {
  epilogue_chunk_general<MODE>(g, stg, lane, t_addr, row0, rows_valid, n0, alpha, bias_vec, cc0,
                               rs_dst, rs_ld, raw_dst, rs_own);
  if constexpr (NCW > 1)
    epilogue_chunk_general<MODE>(g, stg, lane, t_addr, row0, rows_valid, n0, alpha, bias_vec,
                                 cc0 + 1, rs_dst, rs_ld, raw_dst, rs_own);
}

// Epilogue of one tile of the fused reduce-scatter by one warp (see GemmArgs::rs_on).
// blk_row0: first global row of this CTA's 128-row block.  Returns false on a wait that ran
// out.  For a tile of another rank's rows *tflag is the flag to raise with rs_signal_tile
// once the accumulator has been handed back (the stores are only issued here); null for an
// own tile.
template <int BN, int MODE, int NCW>
__device__ __noinline__ bool rs_epilogue_tile(const GemmArgs& g, uint8_t* stg, int lane,
                                                 uint32_t t_addr, int blk_row0, int lane_grp,
                                                 int n0, int nb, float alpha, bool bias_vec,
                                                 int cc0, int epoch, bool& gate_open,
                                                 int** tflag_out) {
  const int R = g.rs_rows_per_rank;
  const int owner = blk_row0 / R;
  const int row0 = blk_row0 + lane_grp * 32;
  if (owner != g.rs.rank) {
    if (!gate_open) {
      if (!rs_wait_gate(g, epoch, lane)) return false;
      gate_open = true;
    }
    __nv_bfloat16* dst = rs_tile_dst(g, blk_row0, lane_grp, n0, tflag_out, nb, g.num_n_blocks);
    epilogue_tile<BN, MODE, NCW>(g, stg, lane, t_addr, row0, 32, n0, alpha, bias_vec, cc0, dst,
                                 g.N);
    return true;
  }
  *tflag_out = nullptr;
  const int lb = (blk_row0 - owner * R) / 128;
  if (!rs_wait_partials(g, lb, nb, g.num_n_blocks, epoch, lane)) return false;
  const __nv_bfloat16* own =
      reinterpret_cast<const __nv_bfloat16*>(static_cast<const char*>(g.rs.heap[g.rs.rank]) +
                                             g.rs_stage_off) +
      (long long)(lb * 128 + lane_grp * 32) * g.N + n0;
  epilogue_tile<BN, MODE, NCW>(g, stg, lane, t_addr, row0, 32, n0, alpha, bias_vec, cc0, nullptr,
                               0, nullptr, own);
  return true;
}

// All eight epilogue warps after the stores of a pushed tile: once every warp has issued its
// stores (named barrier), one thread waits for them to land at the owner (the fence covers
// the other threads' stores through the barrier) and raises the tile's flag there.  The
// other warps go on to the next tile meanwhile.
__device__ __forceinline__ void rs_signal_tile(int* tflag, int epoch, int ew, int lane) {
  asm volatile("bar.sync 1, 256;" ::: "memory");
  if (ew == 0 && lane == 0) {
    __threadfence_system();
    st_release_sys(tflag, epoch);
  }
}

template <int BN, bool A_MN, bool B_MN, int MODE>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                 const __grid_constant__ GemmArgs g) {
  constexpr int B_STAGE_BYTES = BN * BK * 2;
  constexpr int STAGE_BYTES = A_STAGE_BYTES + B_STAGE_BYTES;
  constexpr int STAGES = (BN == 256) ? 4 : 6;
  constexpr uint32_t TMEM_COLS = (2 * BN <= 512) ? ((2 * BN < 32) ? 32 : 2 * BN) : 512;
  static_assert(BN == 64 || BN == 128 || BN == 256, "BN");

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                              ~uintptr_t(1023));
  uint64_t* full_bar =
      reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES + EPI_WARPS * EPI_STAGE_BYTES);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* acc_full = empty_bar + STAGES;
  uint64_t* acc_empty = acc_full + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  constexpr bool COMM = MODE == 1;
  const int ag_ctas = COMM ? g.ag_ctas : 0;
  const bool rs_on = COMM && g.rs_on;
  const int split_k = MODE == 2 ? g.split_k : 1;
  if constexpr (COMM) {
    if ((int)blockIdx.x < ag_ctas) {
      ag_copy_role(g);
      return;
    }
  }
  const int pre = ag_ctas;
  const int cta_id = blockIdx.x - pre, n_ctas = gridDim.x - pre;
  const int rs_epoch = rs_on ? *reinterpret_cast<volatile int*>(g.rs.epoch) + 1 : 0;
  const int ready_target = ag_ctas ? *reinterpret_cast<volatile int*>(g.ag.epoch) + 1
                                   : g.ready_target;
  // with a fused all-gather the local shard's row blocks come first
  // ... and with a fused reduce-scatter the rows owned by the other ranks
  const int mb_shift = ag_ctas ? g.ag.rank * ((g.ag_rows_per_rank + BM - 1) / BM)
                     : rs_on ? ((g.rs.rank + 1) % g.rs.world) * (g.rs_rows_per_rank / BM) : 0;
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int num_tiles = g.num_m_blocks * g.num_n_blocks;
  const int KB = (g.K + BK - 1) / BK;
  const int num_units = num_tiles * split_k;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&acc_full[a], 1);
      mbar_init(&acc_empty[a], EPI_WARPS);
    }
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
    tc_fence_before();
  }
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // The control warpgroup keeps GEMM_CTRL_REGS registers per thread and the epilogue warpgroups take
  // the rest; each setmaxnreg sits inside its own role branch so that no code is reachable
  // from both.
  if (warp < 4) {
    reg_alloc_dec<GEMM_CTRL_REGS>();
  }
  if (warp == 2) {
    if (rs_on && cta_id == 0) rs_open_gate(g, rs_epoch, lane, abort_flag);
  } else if (warp == 0) {
    // ------------------------------------------------------------ producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int u = cta_id; u < num_units && ok; u += n_ctas) {
        const int t = u % num_tiles, ks = u / num_tiles;
        const int kb_lo = ks * KB / split_k, kb_hi = (ks + 1) * KB / split_k;
        int mb, nb;
        tile_coords(t, g.num_m_blocks, g.num_n_blocks, mb_shift, ag_ctas > 0 || rs_on, mb, nb);
        const int m0 = mb * BM, n0 = nb * BN;
        if (g.ready_flags) {
          int f0 = m0 / g.rows_per_flag;
          int m_last = min(m0 + BM, g.M) - 1;
          int f1 = m_last / g.rows_per_flag;
          for (int f = f0; f <= f1 && ok; ++f) {
            if (!wait_flag_ge(g.ready_flags + f, ready_target)) {
              set_error(g.status, abort_flag, NKB_ERR_FLAG_WAIT);
              ok = false;
            }
          }
          if (!ok) break;
          // data landed through the generic proxy of other SMs / GPUs; TMA reads
          // it through the async proxy
          asm volatile("fence.proxy.async.global;" ::: "memory");
        }
        for (int kb = kb_lo; kb < kb_hi; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag)) {
            set_error(g.status, abort_flag, NKB_ERR_EMPTY_WAIT);
            ok = false;
            break;
          }
          uint8_t* sA = smem + stage * STAGE_BYTES;
          uint8_t* sB = sA + A_STAGE_BYTES;
          mbar_expect_tx(&full_bar[stage], STAGE_BYTES);
          if constexpr (!A_MN) {
            tma_load_2d(sA, &tmA, &full_bar[stage], kb * BK, m0);
          } else {
#pragma unroll
            for (int j = 0; j < BM / 64; ++j)
              tma_load_2d(sA + j * (64 * BK * 2), &tmA, &full_bar[stage], m0 + j * 64, kb * BK);
          }
          if constexpr (!B_MN) {
            tma_load_2d(sB, &tmB, &full_bar[stage], kb * BK, n0);
          } else {
#pragma unroll
            for (int j = 0; j < BN / 64; ++j)
              tma_load_2d(sB + j * (64 * BK * 2), &tmB, &full_bar[stage], n0 + j * 64, kb * BK);
          }
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------- MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc_bf16(BM, BN, A_MN ? 1 : 0, B_MN ? 1 : 0);
      const uint64_t dA0 = umma_desc_sw128(smem_u32(smem), A_MN ? 64 * BK * 2 : 16, 1024);
      const uint64_t dB0 =
          umma_desc_sw128(smem_u32(smem) + A_STAGE_BYTES, B_MN ? 64 * BK * 2 : 16, 1024);
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int u = cta_id; u < num_units && ok; u += n_ctas) {
        const int ks = u / num_tiles;
        const int kb_lo = ks * KB / split_k, kb_hi = (ks + 1) * KB / split_k;
        if (!mbar_wait(&acc_empty[acc], acc_phase ^ 1, abort_flag)) {
          set_error(g.status, abort_flag, NKB_ERR_ACC_FREE);
          break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = kb_lo; kb < kb_hi; ++kb) {
          if (!mbar_wait(&full_bar[stage], phase, abort_flag)) {
            set_error(g.status, abort_flag, NKB_ERR_TMA_WAIT);
            ok = false;
            break;
          }
          tc_fence_after();
          // descriptors: only the 14-bit start-address field (16-byte units) changes
          const uint64_t dA = dA0 + (uint32_t)stage * (STAGE_BYTES >> 4);
          const uint64_t dB = dB0 + (uint32_t)stage * (STAGE_BYTES >> 4);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            const uint64_t da = dA + (A_MN ? k * (UMMA_K * 128 >> 4) : k * (UMMA_K * 2 >> 4));
            const uint64_t db = dB + (B_MN ? k * (UMMA_K * 128 >> 4) : k * (UMMA_K * 2 >> 4));
            umma_bf16_ss(d_tmem, da, db, idesc, (kb > kb_lo || k > 0) ? 1u : 0u);
          }
          umma_commit(&empty_bar[stage]);  // frees the stage when these MMAs retire
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (!ok) break;
        umma_commit(&acc_full[acc]);
        if (++acc == 2) {
          acc = 0;
          acc_phase ^= 1;
        }
      }
    }
  } else if (warp >= 4) {
    reg_alloc_inc<GEMM_EPI_REGS>();
    // ------------------------------------------------------------ epilogue
    // Each thread owns one accumulator row (TMEM lane).  Global traffic goes
    // through a per-warp 32-row x 128-byte staging tile so that every global
    // load / store instruction of the warp covers whole 128-byte lines.
    const int lane_grp = warp & 3;  // TMEM lanes this warp may touch: 32*lane_grp ..
    const int ew = warp - 4;        // epilogue warp 0..7
    constexpr int NCW = BN / 128;   // 64-column chunks per warp (two warps share a lane quarter)
    const int cc0 = (ew >> 2) * NCW;
    uint8_t* stg = smem + STAGES * STAGE_BYTES + ew * EPI_STAGE_BYTES;
    int acc = 0;
    uint32_t acc_phase = 0;
    bool rs_gate_open = false;
    const float alpha = g.alpha_dev ? g.alpha * __ldg(g.alpha_dev) : g.alpha;
    const bool bias_vec = g.bias && ((reinterpret_cast<uintptr_t>(g.bias) & 15) == 0);
    const bool fast = MODE == 0 && epi_fast_ok(g);
    long long in_ld;
    const __nv_bfloat16* in_src = epi_async_src(g, &in_ld);
    for (int u = cta_id; u < num_units; u += n_ctas) {
      const int t = u % num_tiles, ks = u / num_tiles;
      int mb, nb;
      tile_coords(t, g.num_m_blocks, g.num_n_blocks, mb_shift, ag_ctas > 0 || rs_on, mb, nb);
      const int row0 = mb * BM + lane_grp * 32;  // first row of this warp's slab
      const int n0 = nb * BN;
      int rows_valid = g.M - row0;
      rows_valid = rows_valid < 0 ? 0 : (rows_valid > 32 ? 32 : rows_valid);
      // the first chunk's residual / saved activation starts moving before the accumulator is ready
      bool first_async = false;
      if (fast && in_src)
        first_async = epi_stage_async(stg, lane, in_src, in_ld, row0, rows_valid, n0 + cc0 * 64, g.N);
      if (!mbar_wait(&acc_full[acc], acc_phase, abort_flag)) {
        set_error(g.status, abort_flag, NKB_ERR_ACC_WAIT);
        break;
      }
      tc_fence_after();
      const uint32_t t_addr = tmem_base + (uint32_t(lane_grp * 32) << 16) + acc * BN;
      int* rs_tflag = nullptr;
      if (rs_on) {
        if (!rs_epilogue_tile<BN, MODE, NCW>(g, stg, lane, t_addr, mb * BM, lane_grp, n0, nb, alpha,
                                             bias_vec, cc0, rs_epoch, rs_gate_open, &rs_tflag)) {
          set_error(g.status, abort_flag, NKB_ERR_FLAG_WAIT);
          break;
        }
      } else if (fast) {
        epilogue_fast_tile(g, stg, lane, t_addr, row0, rows_valid, n0, alpha, bias_vec, cc0, NCW,
                           first_async);
      } else {
        float* raw = MODE == 2 ? g.splitk_ws + ((long long)ks * g.M + row0) * g.N + n0 : nullptr;
        epilogue_tile<BN, MODE, NCW>(g, stg, lane, t_addr, row0, rows_valid, n0, alpha, bias_vec,
                                     cc0, nullptr, 0, raw);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[acc]);
      if (rs_tflag) rs_signal_tile(rs_tflag, rs_epoch, ew, lane);
      if (++acc == 2) {
        acc = 0;
        acc_phase ^= 1;
      }
    }
    if (lane == 0) tma_store_wait<0>();  // bulk stores of this warp have landed
  }

  // ------------------------------------------------------------- teardown
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    if (*abort_flag) {
      // give copies/MMAs that are still in flight time to land before the
      // shared memory and TMEM they target are released
      for (int i = 0; i < 1000; ++i) __nanosleep(1000);
    }
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}


// ------------------------------------------------------------------ CTA-pair kernel
// Two CTAs of a cluster compute one 256 x 256 tile with tcgen05.mma.cta_group::2:
// each CTA loads its own 128 rows of A and its own 128 columns of B (plain per-CTA
// TMA loads whose bytes are counted on the leader's barrier), the leader CTA issues
// the MMAs, which read both CTAs' shared memory, and each CTA's TMEM receives its
// 128 x 256 half of the accumulator.  Operand traffic per FLOP is 2/3 of the
// single-CTA 128 x 256 tile and a stage is 32 KB, so six stages fit.
constexpr int PAIR_STAGES = 6;
constexpr int PAIR_B_BYTES = 128 * BK * 2;
constexpr int PAIR_STAGE_BYTES = A_STAGE_BYTES + PAIR_B_BYTES;

template <bool A_MN, bool B_MN, int MODE>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(GEMM_THREADS, 1)
gemm_bf16_pair_kernel(const __grid_constant__ CUtensorMap tmA,
                      const __grid_constant__ CUtensorMap tmB, const __grid_constant__ GemmArgs g) {
  constexpr int BN = 256;
  constexpr uint32_t TMEM_COLS = 512;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                              ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + PAIR_STAGES * PAIR_STAGE_BYTES +
                                                   EPI_WARPS * EPI_STAGE_BYTES);
  uint64_t* empty_bar = full_bar + PAIR_STAGES;
  uint64_t* acc_full = empty_bar + PAIR_STAGES;
  uint64_t* acc_empty = acc_full + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  constexpr bool COMM = MODE == 1;
  const int ag_ctas = COMM ? g.ag_ctas : 0;
  const bool rs_on = COMM && g.rs_on;
  const int split_k = MODE == 2 ? g.split_k : 1;
  if constexpr (COMM) {
    if ((int)blockIdx.x < ag_ctas) {  // ag_ctas is even: whole clusters take the copy role
      ag_copy_role(g);
      return;
    }
  }
  const int rs_epoch = rs_on ? *reinterpret_cast<volatile int*>(g.rs.epoch) + 1 : 0;
  const int ready_target = ag_ctas ? *reinterpret_cast<volatile int*>(g.ag.epoch) + 1
                                   : g.ready_target;
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;
  const int pre = ag_ctas;
  const int pair = ((int)blockIdx.x - pre) >> 1, npairs = ((int)gridDim.x - pre) >> 1;
  const int num_m2 = (g.M + 255) / 256;
  const int mb_shift = ag_ctas ? g.ag.rank * ((g.ag_rows_per_rank + 255) / 256)
                     : rs_on ? ((g.rs.rank + 1) % g.rs.world) * (g.rs_rows_per_rank / 256) : 0;
  const int num_tiles = num_m2 * g.num_n_blocks;
  const int KB = (g.K + BK - 1) / BK;
  const int num_units = num_tiles * split_k;

  if (threadIdx.x == 0) {
    for (int s = 0; s < PAIR_STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&acc_full[a], 1);
      mbar_init(&acc_empty[a], 2 * EPI_WARPS);  // epilogue warps of both CTAs, leader's copy
    }
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
  }
  if (warp == 1) {
    tmem_alloc_2cta(tmem_slot, TMEM_COLS);
    tmem_relinquish_2cta();
    tc_fence_before();
  }
  __syncthreads();
  cluster_arrive();  // the peer's barriers must exist before anything signals them
  cluster_wait();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  if (warp < 4) {
    reg_alloc_dec<GEMM_CTRL_REGS>();
  }
  if (warp == 2) {
    if (rs_on && pair == 0 && leader) rs_open_gate(g, rs_epoch, lane, abort_flag);
  } else if (warp == 0) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int u = pair; u < num_units && ok; u += npairs) {
        const int t = u % num_tiles, ks = u / num_tiles;
        const int kb_lo = ks * KB / split_k, kb_hi = (ks + 1) * KB / split_k;
        int mb2, nb;
        tile_coords(t, num_m2, g.num_n_blocks, mb_shift, ag_ctas > 0 || rs_on, mb2, nb);
        const int m0 = mb2 * 256 + (int)rank * 128;
        const int nB = nb * BN + (int)rank * 128;
        if (g.ready_flags) {
          if (m0 < g.M) {
            int f0 = m0 / g.rows_per_flag;
            int f1 = (min(m0 + BM, g.M) - 1) / g.rows_per_flag;
            for (int f = f0; f <= f1 && ok; ++f)
              if (!wait_flag_ge(g.ready_flags + f, ready_target)) {
                set_error(g.status, abort_flag, NKB_ERR_FLAG_WAIT);
                ok = false;
              }
          }
          if (!ok) break;
          asm volatile("fence.proxy.async.global;" ::: "memory");
        }
        for (int kb = kb_lo; kb < kb_hi; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag)) {
            set_error(g.status, abort_flag, NKB_ERR_EMPTY_WAIT);
            ok = false;
            break;
          }
          uint8_t* sA = smem + stage * PAIR_STAGE_BYTES;
          uint8_t* sB = sA + A_STAGE_BYTES;
          if (leader) mbar_expect_tx(&full_bar[stage], 2 * PAIR_STAGE_BYTES);
          const uint32_t bar = mapa_shared(smem_u32(&full_bar[stage]), 0);
          if constexpr (!A_MN) {
            tma_load_2d_pair(sA, &tmA, bar, kb * BK, m0);
          } else {
#pragma unroll
            for (int j = 0; j < 2; ++j)
              tma_load_2d_pair(sA + j * (64 * BK * 2), &tmA, bar, m0 + j * 64, kb * BK);
          }
          if constexpr (!B_MN) {
            tma_load_2d_pair(sB, &tmB, bar, kb * BK, nB);
          } else {
#pragma unroll
            for (int j = 0; j < 2; ++j)
              tma_load_2d_pair(sB + j * (64 * BK * 2), &tmB, bar, nB + j * 64, kb * BK);
          }
          if (++stage == PAIR_STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && leader) {
      constexpr uint32_t idesc = umma_idesc_bf16(256, BN, A_MN ? 1 : 0, B_MN ? 1 : 0);
      const uint64_t dA0 = umma_desc_sw128(smem_u32(smem), A_MN ? 64 * BK * 2 : 16, 1024);
      const uint64_t dB0 =
          umma_desc_sw128(smem_u32(smem) + A_STAGE_BYTES, B_MN ? 64 * BK * 2 : 16, 1024);
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int u = pair; u < num_units && ok; u += npairs) {
        const int ks = u / num_tiles;
        const int kb_lo = ks * KB / split_k, kb_hi = (ks + 1) * KB / split_k;
        if (!mbar_wait(&acc_empty[acc], acc_phase ^ 1, abort_flag)) {
          set_error(g.status, abort_flag, NKB_ERR_ACC_FREE);
          break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = kb_lo; kb < kb_hi; ++kb) {
          if (!mbar_wait(&full_bar[stage], phase, abort_flag)) {
            set_error(g.status, abort_flag, NKB_ERR_TMA_WAIT);
            ok = false;
            break;
          }
          tc_fence_after();
          const uint64_t dA = dA0 + (uint32_t)stage * (PAIR_STAGE_BYTES >> 4);
          const uint64_t dB = dB0 + (uint32_t)stage * (PAIR_STAGE_BYTES >> 4);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            const uint64_t da = dA + (A_MN ? k * (UMMA_K * 128 >> 4) : k * (UMMA_K * 2 >> 4));
            const uint64_t db = dB + (B_MN ? k * (UMMA_K * 128 >> 4) : k * (UMMA_K * 2 >> 4));
            umma_bf16_ss_2cta(d_tmem, da, db, idesc, (kb > kb_lo || k > 0) ? 1u : 0u);
          }
          umma_commit_2cta(&empty_bar[stage], 3);  // frees the stage in both CTAs
          if (++stage == PAIR_STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (!ok) break;
        umma_commit_2cta(&acc_full[acc], 3);
        if (++acc == 2) {
          acc = 0;
          acc_phase ^= 1;
        }
      }
    }
  } else if (warp >= 4) {
    reg_alloc_inc<GEMM_EPI_REGS>();
    const int lane_grp = warp & 3;
    const int ew = warp - 4;  // epilogue warp 0..7: two per TMEM lane quarter, 128 columns each
    constexpr int NCW = 2;
    const int cc0 = (ew >> 2) * NCW;
    uint8_t* stg = smem + PAIR_STAGES * PAIR_STAGE_BYTES + ew * EPI_STAGE_BYTES;
    int acc = 0;
    uint32_t acc_phase = 0;
    bool rs_gate_open = false;
    const float alpha = g.alpha_dev ? g.alpha * __ldg(g.alpha_dev) : g.alpha;
    const bool bias_vec = g.bias && ((reinterpret_cast<uintptr_t>(g.bias) & 15) == 0);
    const bool fast = MODE == 0 && epi_fast_ok(g);
    long long in_ld;
    const __nv_bfloat16* in_src = epi_async_src(g, &in_ld);
    for (int u = pair; u < num_units; u += npairs) {
      const int t = u % num_tiles, ks = u / num_tiles;
      int mb2, nb;
      tile_coords(t, num_m2, g.num_n_blocks, mb_shift, ag_ctas > 0 || rs_on, mb2, nb);
      const int row0 = mb2 * 256 + (int)rank * 128 + lane_grp * 32;
      const int n0 = nb * BN;
      int rows_valid = g.M - row0;
      rows_valid = rows_valid < 0 ? 0 : (rows_valid > 32 ? 32 : rows_valid);
      // the first chunk's residual / saved activation starts moving before the accumulator is ready
      bool first_async = false;
      if (fast && in_src)
        first_async = epi_stage_async(stg, lane, in_src, in_ld, row0, rows_valid, n0 + cc0 * 64, g.N);
      if (!mbar_wait(&acc_full[acc], acc_phase, abort_flag)) {
        set_error(g.status, abort_flag, NKB_ERR_ACC_WAIT);
        break;
      }
      tc_fence_after();
      const uint32_t t_addr = tmem_base + (uint32_t(lane_grp * 32) << 16) + acc * BN;
      int* rs_tflag = nullptr;
      if (rs_on) {
        if (!rs_epilogue_tile<BN, MODE, NCW>(g, stg, lane, t_addr, mb2 * 256 + (int)rank * 128,
                                             lane_grp, n0, nb, alpha, bias_vec, cc0, rs_epoch,
                                             rs_gate_open, &rs_tflag)) {
          set_error(g.status, abort_flag, NKB_ERR_FLAG_WAIT);
          break;
        }
      } else if (fast) {
        epilogue_fast_tile(g, stg, lane, t_addr, row0, rows_valid, n0, alpha, bias_vec, cc0, NCW,
                           first_async);
      } else {
        float* raw = MODE == 2 ? g.splitk_ws + ((long long)ks * g.M + row0) * g.N + n0 : nullptr;
        epilogue_tile<BN, MODE, NCW>(g, stg, lane, t_addr, row0, rows_valid, n0, alpha, bias_vec,
                                     cc0, nullptr, 0, raw);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        if (leader) mbar_arrive(&acc_empty[acc]);
        else mbar_arrive_cluster(mapa_shared(smem_u32(&acc_empty[acc]), 0));
      }
      if (rs_tflag) rs_signal_tile(rs_tflag, rs_epoch, ew, lane);
      if (++acc == 2) {
        acc = 0;
        acc_phase ^= 1;
      }
    }
    if (lane == 0) tma_store_wait<0>();  // bulk stores of this warp have landed
  }

  tc_fence_before();
  __syncthreads();
  cluster_arrive();  // neither CTA may leave while the pair's MMAs can still read its smem
  cluster_wait();
  if (warp == 1) {
    if (*abort_flag)
      for (int i = 0; i < 1000; ++i) __nanosleep(1000);
    tc_fence_after();
    tmem_dealloc_2cta(tmem_base, TMEM_COLS);
  }
}

// ------------------------------------------------------------------ host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
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
            cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

// 2-D bf16 tensor map: inner extent `inner` (contiguous), outer extent `outer`
// with a row pitch of `ld` elements; box = box_inner x box_outer, 128B swizzle.
int make_tmap_bf16_2d(CUtensorMap* out, const void* base, long long inner, long long outer,
                      long long ld, int box_inner, int box_outer) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return -1;
  cuuint64_t gdim[2] = {(cuuint64_t)inner, (cuuint64_t)outer};
  cuuint64_t gstride[1] = {(cuuint64_t)ld * 2};
  cuuint32_t box[2] = {(cuuint32_t)box_inner, (cuuint32_t)box_outer};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), gdim, gstride,
                  box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -(int)r - 1000;
}

static int g_num_sms = 0;
static int g_pair_enabled = 1;
static int g_splitk_enabled = 1;
static float* g_splitk_ws = nullptr;      // caller-provided workspace (see nkb_gemm_set_workspace)
static long long g_splitk_ws_floats = 0;  // CTA-pair tiles in the automatic choice
int num_sms() {
  if (!g_num_sms) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&g_num_sms, cudaDevAttrMultiProcessorCount, dev);
    if (g_num_sms <= 0) g_num_sms = 148;
  }
  return g_num_sms;
}

template <int BN, bool A_MN, bool B_MN, int MODE>
static int launch_gemm_mode(const CUtensorMap& tmA, const CUtensorMap& tmB, GemmArgs& g,
                            int max_ctas, cudaStream_t stream) {
  constexpr int STAGES = (BN == 256) ? 4 : 6;
  constexpr int smem_bytes =
      STAGES * (A_STAGE_BYTES + BN * BK * 2) + EPI_WARPS * EPI_STAGE_BYTES + 1024 + 256;
  static bool configured = false;
  auto kern = gemm_bf16_kernel<BN, A_MN, B_MN, MODE>;
  if (!configured) {
    cudaError_t e =
        cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  g.num_m_blocks = (g.M + BM - 1) / BM;
  g.num_n_blocks = (g.N + BN - 1) / BN;
  int tiles = g.num_m_blocks * g.num_n_blocks * g.split_k;
  int ctas = num_sms() - g.ag_ctas;
  if (max_ctas > 0 && max_ctas < ctas) ctas = max_ctas;
  if (tiles < ctas) ctas = tiles;
  g.rs_bn = BN;
  kern<<<ctas + g.ag_ctas, GEMM_THREADS, smem_bytes, stream>>>(tmA, tmB, g);
  return (int)cudaGetLastError();
}

// MODE: 0 plain, 1 fused with a collective, 2 split-K (separate instantiations keep the
// plain kernel free of the other paths' registers and branches)
template <int BN, bool A_MN, bool B_MN>
static int launch_gemm(const CUtensorMap& tmA, const CUtensorMap& tmB, GemmArgs& g, int max_ctas,
                       cudaStream_t stream) {
  if (g.ag_ctas || g.rs_on) return launch_gemm_mode<BN, A_MN, B_MN, 1>(tmA, tmB, g, max_ctas, stream);
  if (g.split_k > 1) return launch_gemm_mode<BN, A_MN, B_MN, 2>(tmA, tmB, g, max_ctas, stream);
  return launch_gemm_mode<BN, A_MN, B_MN, 0>(tmA, tmB, g, max_ctas, stream);
}

template <bool A_MN, bool B_MN, int MODE>
static int launch_gemm_pair_mode(const CUtensorMap& tmA, const CUtensorMap& tmB, GemmArgs& g,
                                 int max_ctas, cudaStream_t stream) {
  constexpr int smem_bytes = PAIR_STAGES * PAIR_STAGE_BYTES + EPI_WARPS * EPI_STAGE_BYTES + 1024 + 256;
  static bool configured = false;
  auto kern = gemm_bf16_pair_kernel<A_MN, B_MN, MODE>;
  if (!configured) {
    cudaError_t e =
        cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  g.num_m_blocks = (g.M + 255) / 256;
  g.num_n_blocks = (g.N + 255) / 256;
  int tiles = g.num_m_blocks * g.num_n_blocks * g.split_k;
  int ctas = num_sms() - g.ag_ctas;
  if (max_ctas > 0 && max_ctas < ctas) ctas = max_ctas;
  ctas &= ~1;
  if (2 * tiles < ctas) ctas = 2 * tiles;
  if (ctas < 2) ctas = 2;
  g.rs_bn = 256;
  kern<<<ctas + g.ag_ctas, GEMM_THREADS, smem_bytes, stream>>>(tmA, tmB, g);
  return (int)cudaGetLastError();
}

template <bool A_MN, bool B_MN>
static int launch_gemm_pair(const CUtensorMap& tmA, const CUtensorMap& tmB, GemmArgs& g,
                            int max_ctas, cudaStream_t stream) {
  if (g.ag_ctas || g.rs_on) return launch_gemm_pair_mode<A_MN, B_MN, 1>(tmA, tmB, g, max_ctas, stream);
  if (g.split_k > 1) return launch_gemm_pair_mode<A_MN, B_MN, 2>(tmA, tmB, g, max_ctas, stream);
  return launch_gemm_pair_mode<A_MN, B_MN, 0>(tmA, tmB, g, max_ctas, stream);
}

}  // namespace nkb

using namespace nkb;

extern "C" void nkb_gemm_set_pair(int enabled) { nkb::g_pair_enabled = enabled; }
extern "C" void nkb_gemm_set_splitk(int enabled) { nkb::g_splitk_enabled = enabled; }
// Caller-owned fp32 workspace for split-K partial tiles (the library never allocates);
// without one, split-K is not used.
extern "C" void nkb_gemm_set_workspace(float* ws, long long n_floats) {
  nkb::g_splitk_ws = ws;
  nkb::g_splitk_ws_floats = n_floats;
}

static int gemm_run_splitk(GemmArgs g, const CUtensorMap& tmA, const CUtensorMap& tmB, int a_mn,
                           int b_mn, bool pair, int BN, int max_ctas, cudaStream_t s) {
  int rc;
  if (pair) {
    rc = (!a_mn && !b_mn) ? launch_gemm_pair<false, false>(tmA, tmB, g, max_ctas, s)
         : (!a_mn && b_mn) ? launch_gemm_pair<false, true>(tmA, tmB, g, max_ctas, s)
         : (a_mn && !b_mn) ? launch_gemm_pair<true, false>(tmA, tmB, g, max_ctas, s)
                           : launch_gemm_pair<true, true>(tmA, tmB, g, max_ctas, s);
  } else if (BN == 256) {
    rc = (!a_mn && !b_mn) ? launch_gemm<256, false, false>(tmA, tmB, g, max_ctas, s)
         : (!a_mn && b_mn) ? launch_gemm<256, false, true>(tmA, tmB, g, max_ctas, s)
         : (a_mn && !b_mn) ? launch_gemm<256, true, false>(tmA, tmB, g, max_ctas, s)
                           : launch_gemm<256, true, true>(tmA, tmB, g, max_ctas, s);
  } else {
    rc = (!a_mn && !b_mn) ? launch_gemm<128, false, false>(tmA, tmB, g, max_ctas, s)
         : (!a_mn && b_mn) ? launch_gemm<128, false, true>(tmA, tmB, g, max_ctas, s)
         : (a_mn && !b_mn) ? launch_gemm<128, true, false>(tmA, tmB, g, max_ctas, s)
                           : launch_gemm<128, true, true>(tmA, tmB, g, max_ctas, s);
  }
  if (rc) return rc;
  const long long MN = (long long)g.M * g.N;
  int blocks = (int)((MN / 4 + 255) / 256);
  if (blocks > 148 * 8) blocks = 148 * 8;
  splitk_reduce_kernel<<<blocks, 256, 0, s>>>(g.splitk_ws, g.split_k, MN, g.N, g.C, g.ldc, g.c_fp32,
                                              g.accumulate, g.alpha, g.alpha_dev);
  return (int)cudaGetLastError();
}

static int gemm_run(GemmArgs g, const void* A, long long lda, int a_mn, const void* B,
                    long long ldb, int b_mn, int max_ctas, int bn_hint, void* stream) {
  const int M = g.M, N = g.N, K = g.K;
  // Tile choice.  bn_hint: 0 = automatic, 128 / 256 = single-CTA tile of that width,
  // 512 = CTA-pair 256 x 256 tile.
  int BN = 256;
  bool pair = false;
  if (bn_hint == 128 || bn_hint == 256) {
    BN = bn_hint;
  } else if (bn_hint == 512) {
    pair = true;
  } else {
    // cost = rounds of the persistent loop x work per round / measured relative
    // throughput of the tile kind (pair 1.0, single-CTA 128x256 0.88, 128x128 0.68)
    int sms = num_sms();
    long long mblk = (M + BM - 1) / BM;
    long long t256 = mblk * ((N + 255) / 256);
    long long t128 = mblk * ((N + 127) / 128);
    double c256 = (double)((t256 + sms - 1) / sms) * 2.0 / 0.88;
    double c128 = (double)((t128 + sms - 1) / sms) * 1.0 / 0.68;
    double best = c256;
    if (N <= 128 || c128 < c256) { BN = 128; best = c128; }
    long long tp = ((M + 255) / 256) * (long long)((N + 255) / 256);
    int npair = sms / 2;
    double cp = (double)((tp + npair - 1) / npair) * 2.0;
    if (g_pair_enabled && M > 128 && N > 128 && cp <= best) pair = true;
    if (g.ag_ctas && (g.ag_rows_per_rank % 256)) pair = false;
  }
  // split-K when the output has too few tiles to occupy the machine and K is long
  g.split_k = 1;
  g.splitk_ws = nullptr;
  if (g_splitk_enabled && g_splitk_ws && !g.ag_ctas && !g.rs_on && g.epi == NKB_EPI_NONE &&
      !g.bias && !g.res && (N % 4) == 0 && (g.ldc % 4) == 0 && K >= 2048) {
    long long slots = pair ? num_sms() / 2 : num_sms();
    long long tl = pair ? ((M + 255) / 256) * (long long)((N + 255) / 256)
                        : ((M + BM - 1) / BM) * (long long)((N + BN - 1) / BN);
    int S = (int)(slots / tl);
    if (S > 8) S = 8;
    while (S > 1 && (K / BK) / S < 8) --S;
    if (S > 1 && tl * 10 <= slots * 7 && (long long)S * M * N <= g_splitk_ws_floats) {
      g.split_k = S;
      g.splitk_ws = g_splitk_ws;
    }
  }
  CUtensorMap tmA, tmB;
  int rc;
  g.tma_c = g.tma_aux = 0;
  if (!g.c_fp32 && !g.ag_ctas && !g.rs_on && g.split_k == 1 && (g.ldc & 7) == 0 &&
      (reinterpret_cast<uintptr_t>(g.C) & 15) == 0 &&
      make_tmap_bf16_2d(&g.tm_c, g.C, N, M, g.ldc, 64, 32) == 0)
    g.tma_c = 1;
  if (g.aux_out && (g.ldaux & 7) == 0 && (reinterpret_cast<uintptr_t>(g.aux_out) & 15) == 0 &&
      make_tmap_bf16_2d(&g.tm_aux, g.aux_out, N, M, g.ldaux, 64, 32) == 0)
    g.tma_aux = 1;
  if (!a_mn) rc = make_tmap_bf16_2d(&tmA, A, K, M, lda, BK, BM);
  else rc = make_tmap_bf16_2d(&tmA, A, M, K, lda, 64, BK);
  if (rc) return rc;
  if (!b_mn) rc = make_tmap_bf16_2d(&tmB, B, K, N, ldb, BK, pair ? 128 : BN);
  else rc = make_tmap_bf16_2d(&tmB, B, N, K, ldb, 64, BK);
  if (rc) return rc;

  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (g.split_k > 1) return gemm_run_splitk(g, tmA, tmB, a_mn, b_mn, pair, BN, max_ctas, s);
  if (pair) {
    if (!a_mn && !b_mn) return launch_gemm_pair<false, false>(tmA, tmB, g, max_ctas, s);
    if (!a_mn && b_mn) return launch_gemm_pair<false, true>(tmA, tmB, g, max_ctas, s);
    if (a_mn && !b_mn) return launch_gemm_pair<true, false>(tmA, tmB, g, max_ctas, s);
    return launch_gemm_pair<true, true>(tmA, tmB, g, max_ctas, s);
  }
#define NKB_DISPATCH(BN_)                                                              \
  if (!a_mn && !b_mn) return launch_gemm<BN_, false, false>(tmA, tmB, g, max_ctas, s); \
  if (!a_mn && b_mn) return launch_gemm<BN_, false, true>(tmA, tmB, g, max_ctas, s);   \
  if (a_mn && !b_mn) return launch_gemm<BN_, true, false>(tmA, tmB, g, max_ctas, s);   \
  return launch_gemm<BN_, true, true>(tmA, tmB, g, max_ctas, s);
  if (BN == 256) { NKB_DISPATCH(256) }
  NKB_DISPATCH(128)
#undef NKB_DISPATCH
}

extern "C" int nkb_gemm_bf16(const void* A, long long lda, int a_mn, const void* B, long long ldb,
                             int b_mn, void* C, long long ldc, int c_fp32, int accumulate, int M,
                             int N, int K, float alpha, const void* bias, const void* res,
                             long long ldres, int epi, void* aux, long long ldaux, int* status,
                             const int* ready_flags, int rows_per_flag, int ready_target,
                             int max_ctas, int bn_hint, const float* alpha_dev, void* stream) {
  if (M <= 0 || N <= 0 || K <= 0) return -2;
  // TMA needs 16-byte aligned bases and row pitches
  if ((lda & 7) || (ldb & 7) || (reinterpret_cast<uintptr_t>(A) & 15) ||
      (reinterpret_cast<uintptr_t>(B) & 15))
    return -3;
  GemmArgs g;
  g.M = M; g.N = N; g.K = K;
  g.C = C; g.ldc = ldc; g.c_fp32 = c_fp32; g.accumulate = accumulate; g.alpha = alpha; g.alpha_dev = alpha_dev;
  g.bias = static_cast<const __nv_bfloat16*>(bias);
  g.res = static_cast<const __nv_bfloat16*>(res);
  g.ldres = ldres;
  g.epi = epi;
  g.aux_out = (epi == NKB_EPI_GELU_FWD) ? static_cast<__nv_bfloat16*>(aux) : nullptr;
  g.aux_in = (epi == NKB_EPI_GELU_BWD) ? static_cast<const __nv_bfloat16*>(aux) : nullptr;
  g.ldaux = ldaux;
  g.status = status;
  g.ready_flags = ready_flags;
  g.rows_per_flag = rows_per_flag > 0 ? rows_per_flag : 1;
  g.ready_target = ready_target;
  g.ag_ctas = 0;
  g.rs_on = 0;
  return gemm_run(g, A, lda, a_mn, B, ldb, b_mn, max_ctas, bn_hint, stream);
}


// A = all-gather over the group of per-rank row shards [rows_per_rank, K] that sit at
// byte offset data_off (row pitch lda) of every member's heap; C = epi(A_full * B^T).
// The gather runs inside the GEMM kernel (see GemmArgs::ag_ctas).  ready_flags: int array
// with one entry per 128-row block of A_full at the same offset of every member's heap
// (zero when the heap is created); A_local: this rank's address of the gather buffer.
extern "C" int nkb_ag_gemm_bf16(void** heap, long long flag_off, long long data_off, int rank,
                                int world, int rows_per_rank, int* epoch, int* ready_flags,
                                int ag_ctas, long long lda, const void* B, long long ldb,
                                int b_mn, void* C, long long ldc, int c_fp32, int N, int K,
                                const void* bias, const void* res, long long ldres, int epi,
                                void* aux, long long ldaux, const void* A_local, int* status,
                                int bn_hint, void* stream) {
  if (world > COMM_MAX_WORLD) return -4;
  if (rows_per_rank % 128) return -5;
  if ((lda & 7) || (ldb & 7) || (data_off & 15)) return -3;
  GemmArgs g;
  g.M = rows_per_rank * world; g.N = N; g.K = K;
  g.C = C; g.ldc = ldc; g.c_fp32 = c_fp32; g.accumulate = 0; g.alpha = 1.f; g.alpha_dev = nullptr;
  g.bias = static_cast<const __nv_bfloat16*>(bias);
  g.res = static_cast<const __nv_bfloat16*>(res);
  g.ldres = ldres;
  g.epi = epi;
  g.aux_out = (epi == NKB_EPI_GELU_FWD) ? static_cast<__nv_bfloat16*>(aux) : nullptr;
  g.aux_in = (epi == NKB_EPI_GELU_BWD) ? static_cast<const __nv_bfloat16*>(aux) : nullptr;
  g.ldaux = ldaux;
  g.status = status;
  g.ready_flags = ready_flags;
  g.rows_per_flag = 128;
  g.ready_target = 0;
  if (ag_ctas <= 0) ag_ctas = 8;
  ag_ctas = (ag_ctas + 1) & ~1;
  g.ag_ctas = world > 1 ? ag_ctas : 0;
  g.rs_on = 0;
  g.ag.heap = heap; g.ag.flag_off = flag_off; g.ag.rank = rank; g.ag.world = world;
  g.ag.epoch = epoch; g.ag.status = status;
  g.ag_data_off = data_off;
  // the flag array lies in the heap too (peers raise the flags): its offset follows from the
  // local addresses of the flags and of the gather buffer
  g.ag_rflag_off = reinterpret_cast<const char*>(ready_flags) -
                   (static_cast<const char*>(A_local) - data_off);
  if (world > 1 && (g.ag_rflag_off < 0 || (g.ag_rflag_off & 3))) return -3;
  g.ag_rows_per_rank = rows_per_rank;
  g.ag_row_bytes = (long long)K * 2;
  g.ag_pitch = lda * 2;
  int rc = gemm_run(g, A_local, lda, 0, B, ldb, b_mn, 0, bn_hint, stream);
  if (rc) return rc;
  if (world > 1) {
    epoch_bump_kernel<<<1, 1, 0, static_cast<cudaStream_t>(stream)>>>(epoch);
    rc = (int)cudaGetLastError();
  }
  return rc;
}

// out[rows_per_rank, N] on every rank = rows [rank*rows_per_rank, ...) of
// sum over ranks of A_r[M, K_r] * B_r[N, K_r]^T (+ bias + res): GEMM and reduce-scatter in
// one kernel (see GemmArgs::rs_on).  stage_off: bf16 [world][rows_per_rank][N] in every
// heap; tflag_off: int [world][rows_per_rank/128][ceil(N/128)] in every heap (zeroed once);
// epoch: device int[4] ([0] completed calls, [2] the go word of this kernel).
extern "C" int nkb_gemm_rs_bf16(void** heap, long long flag_off, long long stage_off,
                                long long tflag_off, int rank, int world, int rows_per_rank,
                                int* epoch, const void* A, long long lda,
                                const void* B, long long ldb, int b_mn, void* out,
                                long long ldout, int N, int K, const void* bias, const void* res,
                                long long ldres, int* status, int bn_hint, void* stream) {
  if (world > COMM_MAX_WORLD) return -4;
  if ((rows_per_rank % 128) || (N % 8)) return -5;
  if ((lda & 7) || (ldb & 7) || (stage_off & 15) || (tflag_off & 3)) return -3;
  GemmArgs g;
  g.M = rows_per_rank * world; g.N = N; g.K = K;
  // bases shifted so that global row numbers (this rank owns rows [rank * R, (rank + 1) * R))
  // index the [R, N] output and residual; only own rows are ever touched through them
  const long long row_shift = (long long)rank * rows_per_rank;
  g.C = static_cast<__nv_bfloat16*>(out) - row_shift * ldout;
  g.ldc = ldout; g.c_fp32 = 0; g.accumulate = 0; g.alpha = 1.f; g.alpha_dev = nullptr;
  g.bias = static_cast<const __nv_bfloat16*>(bias);
  g.res = res ? static_cast<const __nv_bfloat16*>(res) - row_shift * ldres : nullptr;
  g.ldres = ldres;
  g.epi = NKB_EPI_NONE;
  g.aux_out = nullptr; g.aux_in = nullptr; g.ldaux = 0;
  g.status = status;
  g.ready_flags = nullptr; g.rows_per_flag = 1; g.ready_target = 0;
  g.ag_ctas = 0;
  g.rs_on = 1;
  g.rs.heap = heap; g.rs.flag_off = flag_off; g.rs.rank = rank; g.rs.world = world;
  g.rs.epoch = epoch; g.rs.status = status;
  g.rs_stage_off = stage_off; g.rs_tflag_off = tflag_off;
  g.rs_rows_per_rank = rows_per_rank;
  // the tile-flag layout depends on the tile width: fix it (pair tiles when shards are
  // multiples of 256 rows, else single-CTA 128 x 256)
  if (bn_hint == 0) bn_hint = (rows_per_rank % 256 == 0 && g_pair_enabled) ? 512 : 256;
  int rc = gemm_run(g, A, lda, 0, B, ldb, b_mn, 0, bn_hint, stream);
  if (rc) return rc;
  epoch_bump_kernel<<<1, 1, 0, static_cast<cudaStream_t>(stream)>>>(epoch);
  return (int)cudaGetLastError();
}

NKB_DEFINE_WAIT_SETTER(gemm)
