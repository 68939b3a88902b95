// Device-side building blocks of the peer-memory collectives, shared by comm.cu and
// by the GEMM kernels that fuse a collective (gemm_sm100.cu).
#pragma once
#include "ptx.cuh"

namespace nkb {

constexpr int COMM_THREADS = 512;
constexpr int COMM_MAX_CTAS = 160;
constexpr int COMM_MAX_WORLD = 8;
constexpr int COMM_MAX_PEER_UNROLL = 8;

struct CommCtx {
  void* const* heap;   // device array [world] of heap base pointers
  long long flag_off;  // byte offset of the flag region (COMM_MAX_CTAS*COMM_MAX_WORLD ints)
  int rank, world;
  int* epoch;          // device: [0] = completed epochs, [1] = CTAs finished in this call
  int* status;
};

__device__ __forceinline__ int* flag_ptr(const CommCtx& c, int member, int cta, int from) {
  return reinterpret_cast<int*>(static_cast<char*>(c.heap[member]) + c.flag_off) +
         cta * COMM_MAX_WORLD + from;
}

// Cross-rank barrier for this CTA index.  Returns false on timeout.
__device__ __forceinline__ bool cta_barrier(const CommCtx& c, int value) {
  __shared__ int sh_ok;
  __threadfence_system();
  if (threadIdx.x == 0) sh_ok = 1;
  __syncthreads();
  if (threadIdx.x < c.world) {
    const int peer = threadIdx.x;
    st_release_sys(flag_ptr(c, peer, blockIdx.x, c.rank), value);
    if (!wait_flag_ge(flag_ptr(c, c.rank, blockIdx.x, peer), value)) {
      sh_ok = 0;
      if (c.status) atomicCAS(c.status, 0, NKB_ERR_FLAG_WAIT);
    }
  }
  __syncthreads();
  return sh_ok != 0;
}

// The last CTA to finish publishes the new epoch for the next call.
__device__ __forceinline__ void finish_call(const CommCtx& c, int epoch_used) {
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    if (atomicAdd(&c.epoch[1], 1) == (int)gridDim.x - 1) {
      c.epoch[1] = 0;
      c.epoch[0] = epoch_used;
      __threadfence();
    }
  }
}

__device__ __forceinline__ int begin_call(const CommCtx& c) {
  // every CTA reads the epoch before any CTA can finish the call
  return *reinterpret_cast<volatile int*>(c.epoch) + 1;
}

// chunk c of [0, n) split in `parts` pieces aligned to `align` elements
__device__ __forceinline__ void split_range(long long n, int parts, int idx, long long align,
                                            long long& lo, long long& hi) {
  long long per = ((n + parts - 1) / parts + align - 1) / align * align;
  lo = per * idx;
  hi = lo + per;
  if (lo > n) lo = n;
  if (hi > n) hi = n;
}


}  // namespace nkb
