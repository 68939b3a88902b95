// LayerNorm / RMSNorm forward and backward for bf16 activations (fp32 math).
//
// One warp owns a row and keeps it in registers, so the forward reads x once and
// writes y once; the backward reads dy and x once and writes dx once.  Weight /
// bias gradients are column sums produced by nkb_colsum into an fp32 scratch row.
// These replace torch.nn.LayerNorm / RMSNorm calls in the transformer configs;
// the reference itself has no norm kernel.
#include "ptx.cuh"
#include "nkb_api.h"

namespace nkb {

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// NCH chunks of 256 elements (32 lanes x 8 bf16) cover a row of C <= NCH*256.
template <int NCH>
__global__ void __launch_bounds__(128)
norm_fwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                const __nv_bfloat16* __restrict__ b, __nv_bfloat16* __restrict__ y,
                float* __restrict__ stats, int rows, int C, float eps, int rms) {
  const int lane = threadIdx.x & 31;
  const int row = blockIdx.x * 4 + (threadIdx.x >> 5);
  if (row >= rows) return;
  const uint4* xp = reinterpret_cast<const uint4*>(x + (long long)row * C);
  uint4 xv[NCH];
  float sum = 0.f;
#pragma unroll
  for (int c = 0; c < NCH; ++c) {
    const int e = c * 256 + lane * 8;
    if (e < C) {
      xv[c] = ld_nc_v4(xp + c * 32 + lane);
      uint32_t u[4] = {xv[c].x, xv[c].y, xv[c].z, xv[c].w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float2 f = unpack_bf16x2(u[j]);
        sum += f.x + f.y;
      }
    }
  }
  float mean = 0.f;
  if (!rms) mean = warp_sum(sum) / C;
  float var = 0.f;
#pragma unroll
  for (int c = 0; c < NCH; ++c) {
    const int e = c * 256 + lane * 8;
    if (e < C) {
      uint32_t u[4] = {xv[c].x, xv[c].y, xv[c].z, xv[c].w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float2 f = unpack_bf16x2(u[j]);
        float d0 = f.x - mean, d1 = f.y - mean;
        var += d0 * d0 + d1 * d1;
      }
    }
  }
  var = warp_sum(var) / C;
  const float rstd = rsqrtf(var + eps);
  if (lane == 0 && stats) {
    stats[2 * row] = mean;
    stats[2 * row + 1] = rstd;
  }
  uint4* yp = reinterpret_cast<uint4*>(y + (long long)row * C);
  const uint4* wp = reinterpret_cast<const uint4*>(w);
  const uint4* bp = reinterpret_cast<const uint4*>(b);
#pragma unroll
  for (int c = 0; c < NCH; ++c) {
    const int e = c * 256 + lane * 8;
    if (e < C) {
      uint4 wv = __ldg(wp + c * 32 + lane);
      uint4 bv = make_uint4(0, 0, 0, 0);
      if (b) bv = __ldg(bp + c * 32 + lane);
      uint32_t u[4] = {xv[c].x, xv[c].y, xv[c].z, xv[c].w};
      uint32_t wu[4] = {wv.x, wv.y, wv.z, wv.w};
      uint32_t bu[4] = {bv.x, bv.y, bv.z, bv.w};
      uint32_t o[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float2 f = unpack_bf16x2(u[j]);
        float2 wf = unpack_bf16x2(wu[j]);
        float2 bf = unpack_bf16x2(bu[j]);
        o[j] = pack_bf16x2((f.x - mean) * rstd * wf.x + bf.x, (f.y - mean) * rstd * wf.y + bf.y);
      }
      yp[c * 32 + lane] = make_uint4(o[0], o[1], o[2], o[3]);
    }
  }
}

template <int NCH>
__global__ void __launch_bounds__(128)
norm_bwd_dx_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                   const __nv_bfloat16* __restrict__ w, const float* __restrict__ stats,
                   __nv_bfloat16* __restrict__ dx, int rows, int C, int rms,
                   const __nv_bfloat16* __restrict__ dres) {
  // dres (optional): gradient that reaches x along the residual path; added here so that no
  // separate accumulation kernel runs
  const int lane = threadIdx.x & 31;
  const int row = blockIdx.x * 4 + (threadIdx.x >> 5);
  if (row >= rows) return;
  const float mean = rms ? 0.f : stats[2 * row];
  const float rstd = stats[2 * row + 1];
  const uint4* xp = reinterpret_cast<const uint4*>(x + (long long)row * C);
  const uint4* gp = reinterpret_cast<const uint4*>(dy + (long long)row * C);
  const uint4* rp = reinterpret_cast<const uint4*>(dres + (dres ? (long long)row * C : 0));
  const uint4* wp = reinterpret_cast<const uint4*>(w);
  // dyw (dy*w) and xhat kept as packed bf16? keep fp32-exact by recomputing from
  // the cached raw bf16 inputs instead.
  uint4 xv[NCH], gv[NCH];
  float s1 = 0.f, s2 = 0.f;  // sum(dy*w), sum(dy*w*xhat)
#pragma unroll
  for (int c = 0; c < NCH; ++c) {
    const int e = c * 256 + lane * 8;
    if (e < C) {
      xv[c] = ld_nc_v4(xp + c * 32 + lane);
      gv[c] = ld_nc_v4(gp + c * 32 + lane);
      uint4 wv = __ldg(wp + c * 32 + lane);
      uint32_t xu[4] = {xv[c].x, xv[c].y, xv[c].z, xv[c].w};
      uint32_t gu[4] = {gv[c].x, gv[c].y, gv[c].z, gv[c].w};
      uint32_t wu[4] = {wv.x, wv.y, wv.z, wv.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float2 xf = unpack_bf16x2(xu[j]), gf = unpack_bf16x2(gu[j]), wf = unpack_bf16x2(wu[j]);
        float a0 = gf.x * wf.x, a1 = gf.y * wf.y;
        s1 += a0 + a1;
        s2 += a0 * (xf.x - mean) * rstd + a1 * (xf.y - mean) * rstd;
      }
    }
  }
  s1 = rms ? 0.f : warp_sum(s1) / C;
  s2 = warp_sum(s2) / C;
  uint4* op = reinterpret_cast<uint4*>(dx + (long long)row * C);
#pragma unroll
  for (int c = 0; c < NCH; ++c) {
    const int e = c * 256 + lane * 8;
    if (e < C) {
      uint4 wv = __ldg(wp + c * 32 + lane);
      uint4 rv = make_uint4(0, 0, 0, 0);
      if (dres) rv = ld_nc_v4(rp + c * 32 + lane);
      uint32_t xu[4] = {xv[c].x, xv[c].y, xv[c].z, xv[c].w};
      uint32_t gu[4] = {gv[c].x, gv[c].y, gv[c].z, gv[c].w};
      uint32_t wu[4] = {wv.x, wv.y, wv.z, wv.w};
      uint32_t ru[4] = {rv.x, rv.y, rv.z, rv.w};
      uint32_t o[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float2 xf = unpack_bf16x2(xu[j]), gf = unpack_bf16x2(gu[j]), wf = unpack_bf16x2(wu[j]);
        float2 rf = unpack_bf16x2(ru[j]);
        float h0 = (xf.x - mean) * rstd, h1 = (xf.y - mean) * rstd;
        o[j] = pack_bf16x2(rstd * (gf.x * wf.x - s1 - h0 * s2) + rf.x,
                           rstd * (gf.y * wf.y - s1 - h1 * s2) + rf.y);
      }
      op[c * 32 + lane] = make_uint4(o[0], o[1], o[2], o[3]);
    }
  }
}

// Column sums.  Block = 32 x 8 threads: a lane owns 8 adjacent columns (one 16-byte piece
// per row), the 8 warps take interleaved rows; grid = (ceil(C/256), row_splits).
// Each thread streams its pieces through a private ring of COLSUM_RING shared-memory slots
// filled by cp.async (no registers held while in flight, no barriers: a thread only reads
// what it copied itself), so a CTA keeps COLSUM_RING x 4 KB (x2 with the norm input) in
// flight; plain register loads kept only ~1 load per warp outstanding at 2.4 TB/s.
constexpr int COLSUM_RING = 8;
constexpr int COLSUM_UNROLL = COLSUM_RING;  // rows per warp the row split aims for
constexpr int COLSUM_SMEM_BYTES = 2 * COLSUM_RING * 256 * 16;
__device__ __forceinline__ void colsum_cp16(void* smem_dst, const void* gsrc) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(smem_dst)), "l"(gsrc)
               : "memory");
}
__global__ void __launch_bounds__(256)
colsum_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
              const float* __restrict__ stats, float* __restrict__ acc, int rows, int C,
              long long ld, int rms, int* __restrict__ tickets, __nv_bfloat16* __restrict__ out_a,
              __nv_bfloat16* __restrict__ out_b, int accum_a, int accum_b) {
  // ring slots [which: dy | x][slot][thread] (16 bytes each); the reduction buffer reuses it
  extern __shared__ __align__(16) uint8_t colsum_smem[];  // COLSUM_SMEM_BYTES, dynamic
  uint4 (*ring)[COLSUM_RING][256] = reinterpret_cast<uint4 (*)[COLSUM_RING][256]>(colsum_smem);
  float (*sh)[256 + 8] = reinterpret_cast<float (*)[256 + 8]>(colsum_smem);
  const int lane = threadIdx.x & 31, wy = threadIdx.x >> 5;
  const int col = blockIdx.x * 256 + lane * 8;
  float a[8], b[8];
#pragma unroll
  for (int k = 0; k < 8; ++k) a[k] = b[k] = 0.f;
  const bool vec = (col + 8 <= C) && ((ld & 7) == 0) &&
                   ((reinterpret_cast<uintptr_t>(dy) & 15) == 0) &&
                   (!x || (reinterpret_cast<uintptr_t>(x) & 15) == 0);
  const int stride = gridDim.y * 8;
  const int r0 = blockIdx.y * 8 + wy;
  if (col < C && vec) {
    const int n = r0 < rows ? (rows - r0 + stride - 1) / stride : 0;  // rows of this thread
    auto issue = [&](int k) {
      if (k < n) {
        const long long off = (long long)(r0 + (long long)k * stride) * ld + col;
        colsum_cp16(&ring[0][k % COLSUM_RING][threadIdx.x], dy + off);
        if (x) colsum_cp16(&ring[1][k % COLSUM_RING][threadIdx.x], x + off);
      }
      asm volatile("cp.async.commit_group;" ::: "memory");  // one group per step, empty or not
    };
#pragma unroll
    for (int k = 0; k < COLSUM_RING; ++k) issue(k);
    for (int k = 0; k < n; ++k) {
      asm volatile("cp.async.wait_group %0;" ::"n"(COLSUM_RING - 1) : "memory");
      const uint4 gu = ring[0][k % COLSUM_RING][threadIdx.x];
      const uint32_t w[4] = {gu.x, gu.y, gu.z, gu.w};
      if (x) {
        const uint4 xu = ring[1][k % COLSUM_RING][threadIdx.x];
        const uint32_t v[4] = {xu.x, xu.y, xu.z, xu.w};
        const long long rr = r0 + (long long)k * stride;
        const float mean = rms ? 0.f : stats[2 * rr];
        const float rstd = stats[2 * rr + 1];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 f = unpack_bf16x2(w[j]), xf = unpack_bf16x2(v[j]);
          b[2 * j] += f.x;
          b[2 * j + 1] += f.y;
          a[2 * j] += f.x * (xf.x - mean) * rstd;
          a[2 * j + 1] += f.y * (xf.y - mean) * rstd;
        }
      } else {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 f = unpack_bf16x2(w[j]);
          b[2 * j] += f.x;
          b[2 * j + 1] += f.y;
        }
      }
      issue(k + COLSUM_RING);  // refill the slot just read
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
  } else if (col < C) {
    for (int r = r0; r < rows; r += stride) {
      float g[8], xv[8];
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        g[k] = (col + k < C) ? __bfloat162float(dy[(long long)r * ld + col + k]) : 0.f;
        xv[k] = (x && col + k < C) ? __bfloat162float(x[(long long)r * ld + col + k]) : 0.f;
      }
#pragma unroll
      for (int k = 0; k < 8; ++k) b[k] += g[k];
      if (x) {
        const float mean = rms ? 0.f : stats[2 * r];
        const float rstd = stats[2 * r + 1];
#pragma unroll
        for (int k = 0; k < 8; ++k) a[k] += g[k] * (xv[k] - mean) * rstd;
      }
    }
  }
  for (int which = 0; which < 2; ++which) {
    if (which == 0 && !x) continue;
    __syncthreads();
#pragma unroll
    for (int k = 0; k < 8; ++k) sh[wy][lane * 8 + k] = which == 0 ? a[k] : b[k];
    __syncthreads();
    const int c = threadIdx.x;
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) s += sh[i][c];
    const int gc = blockIdx.x * 256 + c;
    if (gc < C) atomicAdd(&acc[(long long)which * C + gc], s);
  }
  if (!tickets) return;
  // Fused finish: the last CTA of a column strip (ticket counter) turns the sums into bf16
  // outputs and leaves the accumulator and the counter at zero for the next call.
  __shared__ int sh_last;
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) sh_last = (atomicAdd(&tickets[blockIdx.x], 1) == (int)gridDim.y - 1);
  __syncthreads();
  if (!sh_last) return;
  __threadfence();
  const int gc = blockIdx.x * 256 + threadIdx.x;
  if (gc < C) {
    for (int which = x ? 0 : 1; which < 2; ++which) {
      float v = atomicExch(&acc[(long long)which * C + gc], 0.f);
      __nv_bfloat16* out = which == 0 ? out_a : out_b;
      if (out) {
        if (which == 0 ? accum_a : accum_b) v += __bfloat162float(out[gc]);
        out[gc] = __float2bfloat16(v);
      }
    }
  }
  if (threadIdx.x == 0) tickets[blockIdx.x] = 0;
}

__global__ void f32_to_bf16_kernel(const float* __restrict__ src, __nv_bfloat16* __restrict__ dst,
                                   long long n, int accumulate) {
  long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (; i < n; i += stride) {
    float v = src[i];
    if (accumulate) v += __bfloat162float(dst[i]);
    dst[i] = __float2bfloat16(v);
  }
}

template <int NCH>
static int launch_fwd(const void* x, const void* w, const void* b, void* y, float* stats, int rows,
                      int C, float eps, int rms, cudaStream_t s) {
  norm_fwd_kernel<NCH><<<(rows + 3) / 4, 128, 0, s>>>(
      static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(w),
      static_cast<const __nv_bfloat16*>(b), static_cast<__nv_bfloat16*>(y), stats, rows, C, eps,
      rms);
  return (int)cudaGetLastError();
}
template <int NCH>
static int launch_bwd(const void* dy, const void* x, const void* w, const float* stats, void* dx,
                      int rows, int C, int rms, const void* dres, cudaStream_t s) {
  norm_bwd_dx_kernel<NCH><<<(rows + 3) / 4, 128, 0, s>>>(
      static_cast<const __nv_bfloat16*>(dy), static_cast<const __nv_bfloat16*>(x),
      static_cast<const __nv_bfloat16*>(w), stats, static_cast<__nv_bfloat16*>(dx), rows, C, rms,
      static_cast<const __nv_bfloat16*>(dres));
  return (int)cudaGetLastError();
}

}  // namespace nkb

using namespace nkb;

#define NKB_NCH_DISPATCH(FN, ...)                          \
  do {                                                     \
    const int nch = (C + 255) / 256;                       \
    if (nch <= 1) return FN<1>(__VA_ARGS__);               \
    if (nch <= 2) return FN<2>(__VA_ARGS__);               \
    if (nch <= 4) return FN<4>(__VA_ARGS__);               \
    if (nch <= 8) return FN<8>(__VA_ARGS__);               \
    if (nch <= 16) return FN<16>(__VA_ARGS__);             \
    if (nch <= 20) return FN<20>(__VA_ARGS__);             \
    if (nch <= 32) return FN<32>(__VA_ARGS__);             \
    return -4;                                             \
  } while (0)

extern "C" int nkb_norm_fwd(const void* x, const void* w, const void* b, void* y, float* stats,
                            int rows, int C, float eps, int rms, void* stream) {
  if (C % 8) return -3;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  NKB_NCH_DISPATCH(launch_fwd, x, w, b, y, stats, rows, C, eps, rms, s);
}

extern "C" int nkb_norm_bwd_dx(const void* dy, const void* x, const void* w, const float* stats,
                               void* dx, int rows, int C, int rms, void* stream) {
  if (C % 8) return -3;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  NKB_NCH_DISPATCH(launch_bwd, dy, x, w, stats, dx, rows, C, rms, nullptr, s);
}

// dx = norm backward of dy + dres (the gradient arriving along the residual connection)
extern "C" int nkb_norm_bwd_dx_res(const void* dy, const void* x, const void* w, const float* stats,
                                   void* dx, int rows, int C, int rms, const void* dres,
                                   void* stream) {
  if (C % 8) return -3;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  NKB_NCH_DISPATCH(launch_bwd, dy, x, w, stats, dx, rows, C, rms, dres, s);
}

// the ring needs more than the 48 KB a kernel gets without opting in (once per device)
static int colsum_configure() {
  static bool done[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return -1;
  if (!done[dev]) {
    if (cudaFuncSetAttribute(nkb::colsum_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             nkb::COLSUM_SMEM_BYTES) != cudaSuccess)
      return -1;
    done[dev] = true;
  }
  return 0;
}

// row splits: about three CTAs per SM (64 KB of ring each), and at least COLSUM_UNROLL rows per
// warp when possible
static int colsum_row_splits(int gx, int rows) {
  int gy = (3 * 148 + gx - 1) / gx;
  int max_gy = rows / (8 * nkb::COLSUM_UNROLL);
  if (max_gy < 1) max_gy = 1;
  if (gy > max_gy) gy = max_gy;
  return gy < 1 ? 1 : gy;
}

extern "C" int nkb_colsum(const void* dy, const void* x, const float* stats, float* acc, int rows,
                          int C, long long ld, int rms, void* stream) {
  if ((C & 1) || (ld & 1)) return -3;
  int gx = (C + 255) / 256;
  int gy = colsum_row_splits(gx, rows);
  if (colsum_configure()) return -6;
  colsum_kernel<<<dim3(gx, gy), 256, nkb::COLSUM_SMEM_BYTES, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(dy), static_cast<const __nv_bfloat16*>(x), stats, acc, rows,
      C, ld, rms, nullptr, nullptr, nullptr, 0, 0);
  return (int)cudaGetLastError();
}

// Column sums straight to bf16 outputs in one launch.  acc: fp32 [2][C] and tickets: int
// [ceil(C/256)], both owned by the caller, zero before the first call and left zero by every
// call (calls that share them must be ordered on one stream).  With x / stats: out_a = sum of
// dy * xhat (norm weight gradient), out_b = sum of dy; without: only out_b.
extern "C" int nkb_colsum_fused(const void* dy, const void* x, const float* stats, float* acc,
                                int* tickets, void* out_a, void* out_b, int accum_a, int accum_b,
                                int rows, int C, long long ld, int rms, void* stream) {
  if ((C & 1) || (ld & 1) || !acc || !tickets) return -3;
  int gx = (C + 255) / 256;
  int gy = colsum_row_splits(gx, rows);
  if (colsum_configure()) return -6;
  colsum_kernel<<<dim3(gx, gy), 256, nkb::COLSUM_SMEM_BYTES, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(dy), static_cast<const __nv_bfloat16*>(x), stats, acc, rows,
      C, ld, rms, tickets, static_cast<__nv_bfloat16*>(out_a), static_cast<__nv_bfloat16*>(out_b),
      accum_a, accum_b);
  return (int)cudaGetLastError();
}

extern "C" int nkb_f32_to_bf16(const float* src, void* dst, long long n, int accumulate,
                               void* stream) {
  if (n <= 0) return 0;
  int blocks = (int)((n + 255) / 256);
  if (blocks > 148 * 8) blocks = 148 * 8;
  f32_to_bf16_kernel<<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      src, static_cast<__nv_bfloat16*>(dst), n, accumulate);
  return (int)cudaGetLastError();
}

// ---------------------------------------------------------------------------
// Allocation-free column sum (declared in nkb_noalloc.h).  The fp32 accumulator
// lives in the library image instead of caller-provided scratch.
#include "nkb_noalloc.h"

static __device__ __align__(256) float g_noalloc_colsum_scratch[2 * NKB_NOALLOC_MAX_COLS];

// Device address of the scratch array per device ordinal.  The array's name is only
// a host-side handle; kernels must be given the address cudaGetSymbolAddress returns
// while the owning device is current.
// Filled on the first call per device.  Two host threads making that first call at the
// same time both store the same address, so the slot is an atomic pointer (no lock needed:
// the look-up is idempotent) and readers never see a torn value.
#include <atomic>
static std::atomic<float*> g_noalloc_scratch_ptr[64];

extern "C" int nkb_colsum_bf16_noalloc(const void* dy, void* out, int rows, int C, long long ld,
                                       void* stream) {
  if (C > NKB_NOALLOC_MAX_COLS) return -4;
  if (C <= 0 || rows <= 0) return -2;
  if ((C & 1) || (ld & 1)) return -3;
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  if (dev < 0 || dev >= 64) return -5;
  float* acc = g_noalloc_scratch_ptr[dev].load(std::memory_order_acquire);
  if (!acc) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_noalloc_colsum_scratch);
    if (e != cudaSuccess) return (int)e;
    acc = static_cast<float*>(p);
    g_noalloc_scratch_ptr[dev].store(acc, std::memory_order_release);
  }
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  // only the plain-sum half [C, 2C) is used; it must start at zero for every call
  e = cudaMemsetAsync(acc + C, 0, sizeof(float) * (size_t)C, s);
  if (e != cudaSuccess) return (int)e;
  int rc = nkb_colsum(dy, nullptr, nullptr, acc, rows, C, ld, 0, stream);
  if (rc) return rc;
  return nkb_f32_to_bf16(acc + C, out, C, 0, stream);
}
