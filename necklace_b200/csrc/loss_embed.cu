// Fused softmax cross-entropy (forward + gradient in place) and token/position
// embedding forward / backward, bf16 activations with fp32 math.
//
// The cross-entropy kernel never materialises fp32 logits or probabilities: one
// block owns a row, stages it in shared memory while it computes the running
// max / sum (single read of the row), then overwrites the row with the gradient.
// The two-phase form (stats, then grad) lets a vocabulary that is split across
// tensor-parallel ranks combine (max, sum, target-logit) with one small
// all-reduce, which is what the reference's VocabParallelEmbedding output path
// needs (necklace/frmwrk/pytorch/mpnn/layers.py:115-131).
#include "ptx.cuh"
#include "nkb_api.h"

namespace nkb {

constexpr int CE_THREADS = 512;

__device__ __forceinline__ void online_combine(float& m, float& s, float m2, float s2) {
  float mn = fmaxf(m, m2);
  if (mn == -INFINITY) { s = 0.f; m = mn; return; }
  s = s * __expf(m - mn) + s2 * __expf(m2 - mn);
  m = mn;
}

__device__ __forceinline__ void block_online_reduce(float& m, float& s, float* sh_m, float* sh_s) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    float m2 = __shfl_xor_sync(0xffffffffu, m, o);
    float s2 = __shfl_xor_sync(0xffffffffu, s, o);
    online_combine(m, s, m2, s2);
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) { sh_m[warp] = m; sh_s[warp] = s; }
  __syncthreads();
  if (warp == 0) {
    const int nw = blockDim.x >> 5;
    float mm = lane < nw ? sh_m[lane] : -INFINITY;
    float ss = lane < nw ? sh_s[lane] : 0.f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      float m2 = __shfl_xor_sync(0xffffffffu, mm, o);
      float s2 = __shfl_xor_sync(0xffffffffu, ss, o);
      online_combine(mm, ss, m2, s2);
    }
    if (lane == 0) { sh_m[0] = mm; sh_s[0] = ss; }
  }
  __syncthreads();
  m = sh_m[0];
  s = sh_s[0];
  __syncthreads();
}

// mode 0: fused fwd+bwd (losses out, grads in place)
// mode 1: stats only  -> stats[t] = (max, sumexp, target logit if owned else 0)
// mode 2: grad only from stats_g[t] = (global max, global sumexp)
template <int MODE>
__global__ void __launch_bounds__(CE_THREADS)
ce_kernel(__nv_bfloat16* __restrict__ logits, const long long* __restrict__ targets,
          float* __restrict__ out, const float* __restrict__ stats_g, int T, int V, long long ld,
          int vocab_start, float grad_scale, int use_smem) {
  extern __shared__ __align__(16) uint8_t ce_smem[];
  __shared__ float sh_m[32], sh_s[32];
  __nv_bfloat16* srow = reinterpret_cast<__nv_bfloat16*>(ce_smem);
  const int t = blockIdx.x;
  if (t >= T) return;
  __nv_bfloat16* row = logits + (long long)t * ld;
  const long long tgt_g = targets[t];
  const int tgt = (tgt_g >= vocab_start && tgt_g < vocab_start + (long long)V)
                      ? (int)(tgt_g - vocab_start) : -1;
  const bool ignore = tgt_g < 0;
  const int V8 = V & ~7;
  const bool vec = ((ld & 7) == 0) && ((reinterpret_cast<uintptr_t>(logits) & 15) == 0);

  float m = -INFINITY, s = 0.f;
  if (MODE != 2) {
    if (vec) {
      for (int i = threadIdx.x * 8; i < V8; i += CE_THREADS * 8) {
        uint4 u = *reinterpret_cast<const uint4*>(row + i);
        if (use_smem) *reinterpret_cast<uint4*>(srow + i) = u;
        uint32_t w[4] = {u.x, u.y, u.z, u.w};
        float f[8];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          float2 p = unpack_bf16x2(w[j]);
          f[2 * j] = p.x; f[2 * j + 1] = p.y;
        }
        float lm = f[0];
#pragma unroll
        for (int j = 1; j < 8; ++j) lm = fmaxf(lm, f[j]);
        float ls = 0.f;
#pragma unroll
        for (int j = 0; j < 8; ++j) ls += __expf(f[j] - lm);
        online_combine(m, s, lm, ls);
      }
      for (int i = V8 + threadIdx.x; i < V; i += CE_THREADS) {
        __nv_bfloat16 b = row[i];
        if (use_smem) srow[i] = b;
        online_combine(m, s, __bfloat162float(b), 1.f);
      }
    } else {
      for (int i = threadIdx.x; i < V; i += CE_THREADS) {
        __nv_bfloat16 b = row[i];
        if (use_smem) srow[i] = b;
        online_combine(m, s, __bfloat162float(b), 1.f);
      }
    }
    block_online_reduce(m, s, sh_m, sh_s);
  } else {
    m = stats_g[2 * t];
    s = stats_g[2 * t + 1];
  }

  if (MODE == 1) {
    if (threadIdx.x == 0) {
      out[3 * t] = m;
      out[3 * t + 1] = s;
      out[3 * t + 2] = tgt >= 0 ? __bfloat162float(row[tgt]) : 0.f;
    }
    return;
  }

  const __nv_bfloat16* src = (MODE == 0 && use_smem) ? srow : row;
  if (MODE == 0 && threadIdx.x == 0) {
    float loss = 0.f;
    if (!ignore && tgt >= 0) loss = (m + __logf(s)) - __bfloat162float(src[tgt]);
    out[t] = loss;
  }
  const float inv = ignore ? 0.f : grad_scale / s;
  const float onehot = ignore ? 0.f : grad_scale;
  const int ldi = (int)(ld < 2147483647LL ? ld : 2147483647LL);
  if (vec) {
    const int Vpad8 = ldi & ~7;
    for (int i = threadIdx.x * 8; i < Vpad8; i += CE_THREADS * 8) {
      uint32_t o[4];
      if (i + 8 <= V) {
        uint4 u = *reinterpret_cast<const uint4*>(src + i);
        uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          float2 p = unpack_bf16x2(w[j]);
          float g0 = __expf(p.x - m) * inv, g1 = __expf(p.y - m) * inv;
          if (i + 2 * j == tgt) g0 -= onehot;
          if (i + 2 * j + 1 == tgt) g1 -= onehot;
          o[j] = pack_bf16x2(g0, g1);
        }
      } else {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          float g0 = 0.f, g1 = 0.f;
          int c0 = i + 2 * j, c1 = c0 + 1;
          if (c0 < V) { g0 = __expf(__bfloat162float(src[c0]) - m) * inv; if (c0 == tgt) g0 -= onehot; }
          if (c1 < V) { g1 = __expf(__bfloat162float(src[c1]) - m) * inv; if (c1 == tgt) g1 -= onehot; }
          o[j] = pack_bf16x2(g0, g1);
        }
      }
      *reinterpret_cast<uint4*>(row + i) = make_uint4(o[0], o[1], o[2], o[3]);
    }
  } else {
    for (int i = threadIdx.x; i < ldi; i += CE_THREADS) {
      float g = 0.f;
      if (i < V) { g = __expf(__bfloat162float(src[i]) - m) * inv; if (i == tgt) g -= onehot; }
      row[i] = __float2bfloat16(g);
    }
  }
}

// out[t, :] = wte[idx[t]-vocab_start, :] (0 if not owned) + wpe[t % S, :]
__global__ void embed_fwd_kernel(const long long* __restrict__ idx,
                                 const __nv_bfloat16* __restrict__ wte,
                                 const __nv_bfloat16* __restrict__ wpe,
                                 __nv_bfloat16* __restrict__ out, int T, int S, int C,
                                 int vocab_start, int vocab_rows) {
  const int t = blockIdx.x;
  if (!NKB_IN_BOUNDS(t, T)) return;
  const long long id = idx[t] - vocab_start;
  const bool owned = id >= 0 && id < vocab_rows;
  const uint4* tp = reinterpret_cast<const uint4*>(wte + (owned ? id : 0) * C);
  const uint4* pp = wpe ? reinterpret_cast<const uint4*>(wpe + (long long)(t % S) * C) : nullptr;
  uint4* op = reinterpret_cast<uint4*>(out + (long long)t * C);
  for (int i = threadIdx.x; i < C / 8; i += blockDim.x) {
    uint4 a = owned ? __ldg(tp + i) : make_uint4(0, 0, 0, 0);
    if (pp) {
      uint4 p = __ldg(pp + i);
      uint32_t au[4] = {a.x, a.y, a.z, a.w}, pu[4] = {p.x, p.y, p.z, p.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float2 x = unpack_bf16x2(au[j]), y = unpack_bf16x2(pu[j]);
        au[j] = pack_bf16x2(x.x + y.x, x.y + y.y);
      }
      a = make_uint4(au[0], au[1], au[2], au[3]);
    }
    op[i] = a;
  }
}

// dwte[idx[t]] += dout[t] (atomic bf16x2) ; one block per token
__global__ void embed_bwd_wte_kernel(const long long* __restrict__ idx,
                                     const __nv_bfloat16* __restrict__ dout,
                                     __nv_bfloat16* __restrict__ dwte, int T, int C,
                                     int vocab_start, int vocab_rows) {
  const int t = blockIdx.x;
  const long long id = idx[t] - vocab_start;
  if (id < 0 || id >= vocab_rows) return;
  const __nv_bfloat162* src = reinterpret_cast<const __nv_bfloat162*>(dout + (long long)t * C);
  __nv_bfloat162* dst = reinterpret_cast<__nv_bfloat162*>(dwte + id * C);
  for (int i = threadIdx.x; i < C / 2; i += blockDim.x) atomicAdd(dst + i, src[i]);
}

// dwpe[s, c] += sum_b dout[b*S + s, c]
__global__ void embed_bwd_wpe_kernel(const __nv_bfloat16* __restrict__ dout,
                                     __nv_bfloat16* __restrict__ dwpe, int T, int S, int C) {
  const int s = blockIdx.x;
  for (int c = threadIdx.x; c < C; c += blockDim.x) {
    float acc = 0.f;
    for (int t = s; t < T; t += S) acc += __bfloat162float(dout[(long long)t * C + c]);
    dwpe[(long long)s * C + c] = __float2bfloat16(__bfloat162float(dwpe[(long long)s * C + c]) + acc);
  }
}

template <int MODE>
static int launch_ce(void* logits, const long long* targets, float* out, const float* stats_g,
                     int T, int V, long long ld, int vocab_start, float grad_scale,
                     cudaStream_t s) {
  size_t smem = 0;
  int use_smem = 0;
  if (MODE == 0) {
    size_t need = ((size_t)V * 2 + 15) & ~size_t(15);
    if (need <= 200 * 1024) {
      smem = need;
      use_smem = 1;
      static size_t configured = 0;
      if (need > 48 * 1024 && need > configured) {
        cudaError_t e = cudaFuncSetAttribute(ce_kernel<MODE>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             200 * 1024);
        if (e != cudaSuccess) return (int)e;
        configured = 200 * 1024;
      }
    }
  }
  ce_kernel<MODE><<<T, CE_THREADS, smem, s>>>(static_cast<__nv_bfloat16*>(logits), targets, out,
                                              stats_g, T, V, ld, vocab_start, grad_scale, use_smem);
  return (int)cudaGetLastError();
}

}  // namespace nkb

using namespace nkb;

extern "C" int nkb_ce_fwd_bwd(void* logits, const long long* targets, float* losses, int T, int V,
                              long long ld, float grad_scale, void* stream) {
  return launch_ce<0>(logits, targets, losses, nullptr, T, V, ld, 0, grad_scale,
                      static_cast<cudaStream_t>(stream));
}
extern "C" int nkb_ce_stats(const void* logits, const long long* targets, float* stats, int T,
                            int V, long long ld, int vocab_start, void* stream) {
  return launch_ce<1>(const_cast<void*>(logits), targets, stats, nullptr, T, V, ld, vocab_start,
                      0.f, static_cast<cudaStream_t>(stream));
}
extern "C" int nkb_ce_grad(void* logits, const long long* targets, const float* stats_g, int T,
                           int V, long long ld, int vocab_start, float grad_scale, void* stream) {
  return launch_ce<2>(logits, targets, nullptr, stats_g, T, V, ld, vocab_start, grad_scale,
                      static_cast<cudaStream_t>(stream));
}
extern "C" int nkb_embed_fwd(const long long* idx, const void* wte, const void* wpe, void* out,
                             int T, int S, int C, int vocab_start, int vocab_rows, void* stream) {
  if (C % 8) return -3;
  embed_fwd_kernel<<<T, 128, 0, static_cast<cudaStream_t>(stream)>>>(
      idx, static_cast<const __nv_bfloat16*>(wte), static_cast<const __nv_bfloat16*>(wpe),
      static_cast<__nv_bfloat16*>(out), T, S, C, vocab_start, vocab_rows);
  return (int)cudaGetLastError();
}
extern "C" int nkb_embed_bwd(const long long* idx, const void* dout, void* dwte, void* dwpe, int T,
                             int S, int C, int vocab_start, int vocab_rows, void* stream) {
  if (C % 2) return -3;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (dwte)
    embed_bwd_wte_kernel<<<T, 128, 0, s>>>(idx, static_cast<const __nv_bfloat16*>(dout),
                                           static_cast<__nv_bfloat16*>(dwte), T, C, vocab_start,
                                           vocab_rows);
  if (dwpe)
    embed_bwd_wpe_kernel<<<S, 256, 0, s>>>(static_cast<const __nv_bfloat16*>(dout),
                                           static_cast<__nv_bfloat16*>(dwpe), T, S, C);
  return (int)cudaGetLastError();
}

NKB_DEFINE_BOUNDS_GETTER(loss)
