// Peer-memory collectives over NVLink / NVSwitch, fused with the math that
// surrounds them.  Every rank maps the same "symmetric heap" of every group
// member; `heap[i]` is the base address of member i's heap in this process and
// buffers are named by byte offsets into it.  Kernels move data with plain
// peer loads / stores (no TMA, no multicast) and synchronise with epoch flags
// that live at `flag_off` in each heap.
//
// Synchronisation scheme: CTA c of a kernel on rank r only ever consumes data
// that CTA c of the same kernel produced on the peers (work is partitioned
// identically on all ranks), so a per-CTA cross-rank barrier is enough and no
// grid-wide sync is needed.  Barriers are "write my epoch into everybody's slot,
// wait until everybody's epoch shows up in mine"; epochs only grow, so flags are
// never reset.  All waits are bounded and report through `status`.
//
// These replace the reference's blocking NCCL calls wrapped in stream syncs
// (necklace/cuda/ncclfns.py:85-260; bucketed all-reduce and reduce-to-owner in
// necklace/frmwrk/pytorch/ptprms.py:256-299, :344-393) and fold the optimizer /
// quantiser into the transfer.
#include "ptx.cuh"
#include "nkb_api.h"
#include "comm_dev.cuh"

namespace nkb {

__global__ void __launch_bounds__(COMM_THREADS) barrier_kernel(CommCtx c) {
  const int e = begin_call(c);
  cta_barrier(c, 2 * e);
  finish_call(c, e);
}

// ------------------------------------------------------------ all-reduce (sum)
// In place on the symmetric buffer at data_off.  Two-shot: rank r reduces shard
// r from all members and stores the result into every member's buffer.
// With `scatter_out` set the reduced shard is written there only (element 0 = first element
// of this rank's shard) and nothing is stored to the peers: a reduce-scatter.
template <bool FP32>
__global__ void __launch_bounds__(COMM_THREADS)
allreduce_kernel(CommCtx c, long long data_off, long long n, float scale, void* scatter_out) {
  const int e = begin_call(c);
  bool ok = cta_barrier(c, 2 * e - 1);
  constexpr int VEC = FP32 ? 4 : 8;  // elements per 16 bytes
  long long s_lo, s_hi;
  split_range(n, c.world, c.rank, VEC * 32, s_lo, s_hi);
  long long lo, hi;
  split_range(s_hi - s_lo, gridDim.x, blockIdx.x, VEC, lo, hi);
  lo += s_lo;
  hi += s_lo;
  const int esz = FP32 ? 4 : 2;
  if (ok) {
    for (long long i = lo + (long long)threadIdx.x * VEC; i < hi; i += COMM_THREADS * VEC) {
      if (i + VEC <= hi) {
        if (!NKB_IN_BOUNDS(i + VEC - 1, n)) continue;
        float acc[VEC];
#pragma unroll
        for (int k = 0; k < VEC; ++k) acc[k] = 0.f;
        for (int p = 0; p < c.world; ++p) {
          const int m = (c.rank + p) % c.world;  // spread the first reads over the peers
          uint4 v = ld_volatile_v4(static_cast<char*>(c.heap[m]) + data_off + i * esz);
          if (FP32) {
            acc[0] += __uint_as_float(v.x); acc[1] += __uint_as_float(v.y);
            acc[2] += __uint_as_float(v.z); acc[3] += __uint_as_float(v.w);
          } else {
            uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int k = 0; k < 4; ++k) {
              float2 f = unpack_bf16x2(u[k]);
              acc[2 * k] += f.x;
              acc[2 * k + 1] += f.y;
            }
          }
        }
        uint4 o;
        if (FP32) {
          o = make_uint4(__float_as_uint(acc[0] * scale), __float_as_uint(acc[1] * scale),
                         __float_as_uint(acc[2] * scale), __float_as_uint(acc[3] * scale));
        } else {
          o = make_uint4(pack_bf16x2(acc[0] * scale, acc[1] * scale),
                         pack_bf16x2(acc[2] * scale, acc[3] * scale),
                         pack_bf16x2(acc[4] * scale, acc[5] * scale),
                         pack_bf16x2(acc[6] * scale, acc[7] * scale));
        }
        if (scatter_out) {
          *reinterpret_cast<uint4*>(static_cast<char*>(scatter_out) + (i - s_lo) * esz) = o;
        } else {
          for (int p = 0; p < c.world; ++p) {
            const int m = (c.rank + p) % c.world;
            *reinterpret_cast<uint4*>(static_cast<char*>(c.heap[m]) + data_off + i * esz) = o;
          }
        }
      } else {
        for (long long j = i; j < hi; ++j) {
          float acc = 0.f;
          for (int m = 0; m < c.world; ++m) {
            const char* src = static_cast<const char*>(c.heap[m]) + data_off + j * esz;
            acc += FP32 ? *reinterpret_cast<const volatile float*>(src)
                        : __bfloat162float(*reinterpret_cast<const volatile __nv_bfloat16*>(src));
          }
          acc *= scale;
          for (int m = 0; m < (scatter_out ? 1 : c.world); ++m) {
            char* dst = scatter_out ? static_cast<char*>(scatter_out) + (j - s_lo) * esz
                                    : static_cast<char*>(c.heap[m]) + data_off + j * esz;
            if (FP32) *reinterpret_cast<float*>(dst) = acc;
            else *reinterpret_cast<__nv_bfloat16*>(dst) = __float2bfloat16(acc);
          }
        }
      }
    }
    cta_barrier(c, 2 * e);
  }
  finish_call(c, e);
}

// ----------------------------------------------------------------- all-gather
// Member r's shard lives at data_off + r*shard_bytes in its own heap; after the
// call every member holds all shards.  Each rank pushes its shard to the peers.
__global__ void __launch_bounds__(COMM_THREADS)
allgather_kernel(CommCtx c, long long data_off, long long shard_bytes) {
  const int e = begin_call(c);
  bool ok = cta_barrier(c, 2 * e - 1);  // peers finished reading what we overwrite
  if (ok) {
    const long long n16 = shard_bytes >> 4;
    long long lo, hi;
    split_range(n16, gridDim.x, blockIdx.x, 1, lo, hi);
    const long long off = data_off + (long long)c.rank * shard_bytes;
    const uint4* src = reinterpret_cast<const uint4*>(static_cast<char*>(c.heap[c.rank]) + off);
    for (long long i = lo + threadIdx.x; i < hi; i += COMM_THREADS) {
      uint4 v = src[i];
      for (int p = 1; p < c.world; ++p) {
        const int m = (c.rank + p) % c.world;
        reinterpret_cast<uint4*>(static_cast<char*>(c.heap[m]) + off)[i] = v;
      }
    }
    cta_barrier(c, 2 * e);
  }
  finish_call(c, e);
}

// ------------------------------------------------------------------ broadcast
// The root's bytes at data_off are pushed to the same offset of every other member
// (the input batch / shape broadcast over a tensor-parallel group).
__global__ void __launch_bounds__(COMM_THREADS)
bcast_kernel(CommCtx c, long long data_off, long long nbytes, int root) {
  const int e = begin_call(c);
  bool ok = cta_barrier(c, 2 * e - 1);  // receivers are done with the previous content
  if (ok) {
    if (c.rank == root) {
      const long long n16 = nbytes >> 4;
      long long lo, hi;
      split_range(n16, gridDim.x, blockIdx.x, 1, lo, hi);
      const uint4* src =
          reinterpret_cast<const uint4*>(static_cast<char*>(c.heap[c.rank]) + data_off);
      for (long long i = lo + threadIdx.x; i < hi; i += COMM_THREADS) {
        uint4 v = src[i];
        for (int p = 1; p < c.world; ++p) {
          const int m = (c.rank + p) % c.world;
          reinterpret_cast<uint4*>(static_cast<char*>(c.heap[m]) + data_off)[i] = v;
        }
      }
    }
    cta_barrier(c, 2 * e);
  }
  finish_call(c, e);
}

// ------------------------------------------ 2-bit compressed gradient all-reduce
// g (+ residual) -> 2-bit codes (error feedback kept in `residual`) in this
// rank's code buffer; rank r then sums the codes of shard r from all members
// into int8 counts (n_plus - n_minus, exact) and pushes the counts to every
// member; finally every rank decodes counts * thr * scale into `out`.
// NVLink traffic per rank: n/4 bytes of codes in + n bytes of counts out, versus
// 8n for an fp32 ring all-reduce.
// Work split: CTA c owns sub-slice c of *every* shard, so each phase only reads
// what the same CTA index produced on the peers.
struct QuantArgs {
  const void* g;
  int g_fp32;
  float* residual;
  long long codes_off;   // uint32 [ceil(n/16)]
  long long counts_off;  // int8 [n] (padded to 16)
  void* out;
  int out_fp32;
  long long n;
  float thr, scale;
};

__device__ __forceinline__ uint32_t q2_code(float a, float thr, float& resid) {
  if (a >= thr) { resid = a - thr; return 1u; }
  if (a <= -thr) { resid = a + thr; return 2u; }
  resid = a;
  return 0u;
}

__global__ void __launch_bounds__(COMM_THREADS)
dp_quant_allreduce_kernel(CommCtx c, QuantArgs q) {
  const int e = begin_call(c);
  const long long nwords = (q.n + 15) >> 4;
  uint32_t* my_codes = reinterpret_cast<uint32_t*>(static_cast<char*>(c.heap[c.rank]) + q.codes_off);

  // phase 0: quantise my sub-slice of every shard (word granularity)
  for (int s = 0; s < c.world; ++s) {
    long long s_lo, s_hi, lo, hi;
    split_range(nwords, c.world, s, 4, s_lo, s_hi);
    split_range(s_hi - s_lo, gridDim.x, blockIdx.x, 4, lo, hi);
    lo += s_lo;
    hi += s_lo;
    for (long long w = lo + threadIdx.x; w < hi; w += COMM_THREADS) {
      const long long base = w << 4;
      uint32_t word = 0;
#pragma unroll 4
      for (int i = 0; i < 16; ++i) {
        const long long idx = base + i;
        if (idx < q.n) {
          float gval = q.g_fp32 ? static_cast<const float*>(q.g)[idx]
                                : __bfloat162float(static_cast<const __nv_bfloat16*>(q.g)[idx]);
          float res;
          uint32_t code = q2_code(gval + q.residual[idx], q.thr, res);
          q.residual[idx] = res;
          word |= code << (2 * i);
        }
      }
      my_codes[w] = word;
    }
  }
  bool ok = cta_barrier(c, 2 * e - 1);

  // phase 1: counts for my shard, pushed to everybody
  if (ok) {
    long long s_lo, s_hi, lo, hi;
    split_range(nwords, c.world, c.rank, 4, s_lo, s_hi);
    split_range(s_hi - s_lo, gridDim.x, blockIdx.x, 4, lo, hi);
    lo += s_lo;
    hi += s_lo;
    for (long long w = lo + threadIdx.x; w < hi; w += COMM_THREADS) {
      int cnt[16];
#pragma unroll
      for (int i = 0; i < 16; ++i) cnt[i] = 0;
      for (int p = 0; p < c.world; ++p) {
        const int m = (c.rank + p) % c.world;
        const uint32_t word = *reinterpret_cast<const volatile uint32_t*>(
            static_cast<const char*>(c.heap[m]) + q.codes_off + w * 4);
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const uint32_t code = (word >> (2 * i)) & 3u;
          cnt[i] += (code == 1u) - (code == 2u);
        }
      }
      uint4 packed;
      uint32_t pw[4];
#pragma unroll
      for (int k = 0; k < 4; ++k)
        pw[k] = (uint32_t(cnt[4 * k] & 0xff)) | (uint32_t(cnt[4 * k + 1] & 0xff) << 8) |
                (uint32_t(cnt[4 * k + 2] & 0xff) << 16) | (uint32_t(cnt[4 * k + 3] & 0xff) << 24);
      packed = make_uint4(pw[0], pw[1], pw[2], pw[3]);
      for (int p = 0; p < c.world; ++p) {
        const int m = (c.rank + p) % c.world;
        *reinterpret_cast<uint4*>(static_cast<char*>(c.heap[m]) + q.counts_off + w * 16) = packed;
      }
    }
    ok = cta_barrier(c, 2 * e);
  }

  // phase 2: decode every shard's sub-slice (written by CTA index == mine on the owners)
  if (ok) {
    const float mul = q.thr * q.scale;
    const char* counts = static_cast<const char*>(c.heap[c.rank]) + q.counts_off;
    for (int s = 0; s < c.world; ++s) {
      long long s_lo, s_hi, lo, hi;
      split_range(nwords, c.world, s, 4, s_lo, s_hi);
      split_range(s_hi - s_lo, gridDim.x, blockIdx.x, 4, lo, hi);
      lo += s_lo;
      hi += s_lo;
      for (long long w = lo + threadIdx.x; w < hi; w += COMM_THREADS) {
        uint4 pk = ld_volatile_v4(counts + w * 16);
        uint32_t pw[4] = {pk.x, pk.y, pk.z, pk.w};
        const long long base = w << 4;
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const long long idx = base + i;
          if (idx < q.n) {
            const int cnt = (int)(signed char)((pw[i >> 2] >> (8 * (i & 3))) & 0xff);
            const float v = cnt * mul;
            if (q.out_fp32) static_cast<float*>(q.out)[idx] = v;
            else static_cast<__nv_bfloat16*>(q.out)[idx] = __float2bfloat16(v);
          }
        }
      }
    }
  }
  finish_call(c, e);
}

// ------------------------------- ZeRO: reduce-scatter + optimizer + all-gather
// Gradients (bf16, n_total elements, padded so that n_total % world == 0 and the
// shard is a multiple of 8) sit at grad_off in every heap; the bf16 parameters
// at param_off.  Rank r sums shard r of the gradients from all members in fp32,
// applies the optimizer to its fp32 master shard and stores the new bf16
// parameters into every member's parameter buffer.  One kernel replaces
// reduce(-scatter), the optimizer step and the parameter broadcast / all-gather.
struct OptArgs {
  long long grad_off, param_off;
  long long n_total;
  float* master;
  float* s1;  // adam m / sgd momentum
  float* s2;  // adam v
  float lr, beta1, beta2, eps, wd, c1, c2, gscale;
  int adam;        // 1 = Adam(W), 0 = SGD momentum
  int first_step;  // SGD: momentum buffer initialised from the gradient
  const float* hyper;  // optional device floats {lr, c1, c2, t, gmul}: override lr, c1, c2; gmul scales gscale
};

__global__ void __launch_bounds__(COMM_THREADS)
rs_opt_ag_kernel(CommCtx c, OptArgs o) {
  if (o.hyper) { o.lr = o.hyper[0]; o.c1 = o.hyper[1]; o.c2 = o.hyper[2]; o.gscale *= o.hyper[4]; }
  const int e = begin_call(c);
  bool ok = cta_barrier(c, 2 * e - 1);  // everyone's gradients are complete
  if (ok) {
    const long long shard = o.n_total / c.world;
    const long long s_lo = shard * c.rank;
    long long lo, hi;
    split_range(shard, gridDim.x, blockIdx.x, 8, lo, hi);
    // Peer loads are latency bound (~2-3 us over NVLink): keep two iterations of
    // `world` 16-byte loads in flight per thread.
    uint4 nxt[COMM_MAX_PEER_UNROLL];
    auto load_all = [&](long long i, uint4* v) {
#pragma unroll
      for (int p = 0; p < COMM_MAX_PEER_UNROLL; ++p) {
        if (p < c.world) {
          const int m = (c.rank + p) % c.world;
          v[p] = ld_volatile_v4(static_cast<const char*>(c.heap[m]) + o.grad_off + (s_lo + i) * 2);
        }
      }
    };
    const long long i_first = lo + (long long)threadIdx.x * 8;
    if (i_first < hi) load_all(i_first, nxt);
    for (long long i = i_first; i < hi; i += COMM_THREADS * 8) {
      if (!NKB_IN_BOUNDS(s_lo + i + 7, o.n_total)) break;
      uint4 cur[COMM_MAX_PEER_UNROLL];
#pragma unroll
      for (int p = 0; p < COMM_MAX_PEER_UNROLL; ++p) cur[p] = nxt[p];
      if (i + COMM_THREADS * 8 < hi) load_all(i + COMM_THREADS * 8, nxt);
      float g[8];
#pragma unroll
      for (int k = 0; k < 8; ++k) g[k] = 0.f;
#pragma unroll
      for (int p = 0; p < COMM_MAX_PEER_UNROLL; ++p) {
        if (p < c.world) {
          uint32_t u[4] = {cur[p].x, cur[p].y, cur[p].z, cur[p].w};
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            float2 f = unpack_bf16x2(u[k]);
            g[2 * k] += f.x;
            g[2 * k + 1] += f.y;
          }
        }
      }
      float4 p0 = reinterpret_cast<float4*>(o.master + i)[0];
      float4 p1 = reinterpret_cast<float4*>(o.master + i)[1];
      float pa[8] = {p0.x, p0.y, p0.z, p0.w, p1.x, p1.y, p1.z, p1.w};
      if (o.adam) {
        float4 m0 = reinterpret_cast<float4*>(o.s1 + i)[0], m1 = reinterpret_cast<float4*>(o.s1 + i)[1];
        float4 v0 = reinterpret_cast<float4*>(o.s2 + i)[0], v1 = reinterpret_cast<float4*>(o.s2 + i)[1];
        float ma[8] = {m0.x, m0.y, m0.z, m0.w, m1.x, m1.y, m1.z, m1.w};
        float va[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          const float gk = g[k] * o.gscale;
          ma[k] = o.beta1 * ma[k] + (1.f - o.beta1) * gk;
          va[k] = o.beta2 * va[k] + (1.f - o.beta2) * gk * gk;
          const float upd = (ma[k] * o.c1) / (sqrtf(va[k] * o.c2) + o.eps);
          pa[k] -= o.lr * (upd + o.wd * pa[k]);
        }
        reinterpret_cast<float4*>(o.s1 + i)[0] = make_float4(ma[0], ma[1], ma[2], ma[3]);
        reinterpret_cast<float4*>(o.s1 + i)[1] = make_float4(ma[4], ma[5], ma[6], ma[7]);
        reinterpret_cast<float4*>(o.s2 + i)[0] = make_float4(va[0], va[1], va[2], va[3]);
        reinterpret_cast<float4*>(o.s2 + i)[1] = make_float4(va[4], va[5], va[6], va[7]);
      } else {
        float ma[8];
        if (o.s1) {
          float4 m0 = reinterpret_cast<float4*>(o.s1 + i)[0], m1 = reinterpret_cast<float4*>(o.s1 + i)[1];
          ma[0] = m0.x; ma[1] = m0.y; ma[2] = m0.z; ma[3] = m0.w;
          ma[4] = m1.x; ma[5] = m1.y; ma[6] = m1.z; ma[7] = m1.w;
        }
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          float gk = g[k] * o.gscale + o.wd * pa[k];
          if (o.s1) {
            ma[k] = o.first_step ? gk : (o.beta1 * ma[k] + gk);
            gk = ma[k];
          }
          pa[k] -= o.lr * gk;
        }
        if (o.s1) {
          reinterpret_cast<float4*>(o.s1 + i)[0] = make_float4(ma[0], ma[1], ma[2], ma[3]);
          reinterpret_cast<float4*>(o.s1 + i)[1] = make_float4(ma[4], ma[5], ma[6], ma[7]);
        }
      }
      reinterpret_cast<float4*>(o.master + i)[0] = make_float4(pa[0], pa[1], pa[2], pa[3]);
      reinterpret_cast<float4*>(o.master + i)[1] = make_float4(pa[4], pa[5], pa[6], pa[7]);
      const uint4 pb = make_uint4(pack_bf16x2(pa[0], pa[1]), pack_bf16x2(pa[2], pa[3]),
                                  pack_bf16x2(pa[4], pa[5]), pack_bf16x2(pa[6], pa[7]));
      for (int p = 0; p < c.world; ++p) {
        const int m = (c.rank + p) % c.world;
        *reinterpret_cast<uint4*>(static_cast<char*>(c.heap[m]) + o.param_off + (s_lo + i) * 2) = pb;
      }
    }
    cta_barrier(c, 2 * e);  // all parameter shards have landed everywhere
  }
  finish_call(c, e);
}

static int comm_grid(int max_ctas, long long work_items) {
  int g = max_ctas > 0 ? max_ctas : 148;
  if (g > COMM_MAX_CTAS) g = COMM_MAX_CTAS;
  long long need = (work_items + COMM_THREADS - 1) / COMM_THREADS;
  if (need < 1) need = 1;
  if (g > need) g = (int)need;
  return g;
}

}  // namespace nkb

using namespace nkb;

static CommCtx make_ctx(void** heap, long long flag_off, int rank, int world, int* epoch,
                        int* status) {
  CommCtx c;
  c.heap = heap; c.flag_off = flag_off; c.rank = rank; c.world = world; c.epoch = epoch;
  c.status = status;
  return c;
}

extern "C" int nkb_comm_flag_bytes(void) { return COMM_MAX_CTAS * COMM_MAX_WORLD * 4; }

extern "C" int nkb_comm_barrier(void** heap, long long flag_off, int rank, int world, int* epoch,
                                int* status, void* stream) {
  if (world > COMM_MAX_WORLD) return -4;
  barrier_kernel<<<1, COMM_THREADS, 0, static_cast<cudaStream_t>(stream)>>>(
      make_ctx(heap, flag_off, rank, world, epoch, status));
  return (int)cudaGetLastError();
}

extern "C" int nkb_comm_allreduce(void** heap, long long flag_off, long long data_off, long long n,
                                  int fp32, float scale, int rank, int world, int* epoch,
                                  int* status, int max_ctas, void* stream) {
  if (world > COMM_MAX_WORLD) return -4;
  if (data_off & 15) return -3;
  CommCtx c = make_ctx(heap, flag_off, rank, world, epoch, status);
  int grid = comm_grid(max_ctas, n / world / (fp32 ? 4 : 8));
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (fp32) allreduce_kernel<true><<<grid, COMM_THREADS, 0, s>>>(c, data_off, n, scale, nullptr);
  else allreduce_kernel<false><<<grid, COMM_THREADS, 0, s>>>(c, data_off, n, scale, nullptr);
  return (int)cudaGetLastError();
}

// Reduce-scatter: rank r receives the sum over members of elements [r*n/world, (r+1)*n/world)
// of the symmetric buffer at data_off, times scale, in `out` (any device memory of this rank).
// n must be a multiple of world * 256 elements so that the shards are equal.
extern "C" int nkb_comm_reduce_scatter(void** heap, long long flag_off, long long data_off,
                                       long long n, int fp32, float scale, void* out, int rank,
                                       int world, int* epoch, int* status, int max_ctas,
                                       void* stream) {
  if (world > COMM_MAX_WORLD) return -4;
  if ((data_off & 15) || (reinterpret_cast<uintptr_t>(out) & 15) || out == nullptr) return -3;
  if (n % (256LL * world)) return -3;
  CommCtx c = make_ctx(heap, flag_off, rank, world, epoch, status);
  int grid = comm_grid(max_ctas, n / world / (fp32 ? 4 : 8));
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (fp32) allreduce_kernel<true><<<grid, COMM_THREADS, 0, s>>>(c, data_off, n, scale, out);
  else allreduce_kernel<false><<<grid, COMM_THREADS, 0, s>>>(c, data_off, n, scale, out);
  return (int)cudaGetLastError();
}

extern "C" int nkb_comm_bcast(void** heap, long long flag_off, long long data_off,
                              long long nbytes, int root, int rank, int world, int* epoch,
                              int* status, int max_ctas, void* stream) {
  if (world > COMM_MAX_WORLD) return -4;
  if ((data_off & 15) || (nbytes & 15) || root < 0 || root >= world) return -3;
  CommCtx c = make_ctx(heap, flag_off, rank, world, epoch, status);
  int grid = comm_grid(max_ctas, nbytes / 16);
  bcast_kernel<<<grid, COMM_THREADS, 0, static_cast<cudaStream_t>(stream)>>>(c, data_off, nbytes,
                                                                            root);
  return (int)cudaGetLastError();
}

extern "C" int nkb_comm_allgather(void** heap, long long flag_off, long long data_off,
                                  long long shard_bytes, int rank, int world, int* epoch,
                                  int* status, int max_ctas, void* stream) {
  if (world > COMM_MAX_WORLD) return -4;
  if ((data_off & 15) || (shard_bytes & 15)) return -3;
  CommCtx c = make_ctx(heap, flag_off, rank, world, epoch, status);
  int grid = comm_grid(max_ctas, shard_bytes / 16);
  allgather_kernel<<<grid, COMM_THREADS, 0, static_cast<cudaStream_t>(stream)>>>(c, data_off,
                                                                                shard_bytes);
  return (int)cudaGetLastError();
}

extern "C" int nkb_comm_dp_quant_allreduce(void** heap, long long flag_off, const void* g,
                                           int g_fp32, float* residual, long long codes_off,
                                           long long counts_off, void* out, int out_fp32,
                                           long long n, float thr, float scale, int rank,
                                           int world, int* epoch, int* status, int max_ctas,
                                           void* stream) {
  if (world > COMM_MAX_WORLD) return -4;
  if ((codes_off & 15) || (counts_off & 15)) return -3;
  CommCtx c = make_ctx(heap, flag_off, rank, world, epoch, status);
  QuantArgs q;
  q.g = g; q.g_fp32 = g_fp32; q.residual = residual; q.codes_off = codes_off;
  q.counts_off = counts_off; q.out = out; q.out_fp32 = out_fp32; q.n = n; q.thr = thr;
  q.scale = scale;
  int grid = comm_grid(max_ctas, (n + 15) / 16 / world);
  dp_quant_allreduce_kernel<<<grid, COMM_THREADS, 0, static_cast<cudaStream_t>(stream)>>>(c, q);
  return (int)cudaGetLastError();
}

extern "C" int nkb_comm_rs_opt_ag(void** heap, long long flag_off, long long grad_off,
                                  long long param_off, long long n_total, float* master, float* s1,
                                  float* s2, int adam, float lr, float beta1, float beta2,
                                  float eps, float wd, float c1, float c2, float gscale,
                                  int first_step, const float* hyper_dev, int rank, int world,
                                  int* epoch, int* status, int max_ctas, void* stream) {
  if (world > COMM_MAX_WORLD) return -4;
  if ((grad_off & 15) || (param_off & 15) || (n_total % (8LL * world))) return -3;
  CommCtx c = make_ctx(heap, flag_off, rank, world, epoch, status);
  OptArgs o;
  o.grad_off = grad_off; o.param_off = param_off; o.n_total = n_total; o.master = master;
  o.s1 = s1; o.s2 = s2; o.lr = lr; o.beta1 = beta1; o.beta2 = beta2; o.eps = eps; o.wd = wd;
  o.c1 = c1; o.c2 = c2; o.gscale = gscale; o.adam = adam; o.first_step = first_step; o.hyper = hyper_dev;
  int grid = comm_grid(max_ctas, n_total / world / 8);
  rs_opt_ag_kernel<<<grid, COMM_THREADS, 0, static_cast<cudaStream_t>(stream)>>>(c, o);
  return (int)cudaGetLastError();
}

NKB_DEFINE_WAIT_SETTER(comm)
NKB_DEFINE_BOUNDS_GETTER(comm)
