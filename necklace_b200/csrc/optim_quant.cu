// Flat-buffer optimizers (Adam/AdamW, SGD-momentum), the 2-bit threshold
// gradient codec with error feedback, and small flat helpers.
//
// The codec reproduces the arithmetic of the reference's two numba kernels
// (necklace/cuda/quantize.py:16-91): a value >= thr encodes as 01 and decodes to
// +thr, a value <= -thr encodes as 10 and decodes to -thr, everything else is 00
// and decodes to 0; sixteen codes share a uint32 with element i at bits
// [2i, 2i+2).  Unlike the reference kernels these cover inputs of any size
// (grid-stride) and add the previous residual before coding, so the caller no
// longer has to implement error feedback itself.
#include "ptx.cuh"
#include "nkb_api.h"

namespace nkb {

__device__ __forceinline__ float load_as_float(const void* p, long long i, int fp32) {
  return fp32 ? static_cast<const float*>(p)[i]
              : __bfloat162float(static_cast<const __nv_bfloat16*>(p)[i]);
}

// 4 elements per thread-iteration, 16-byte accesses on the fp32 state.
__global__ void __launch_bounds__(256)
adam_flat_kernel(float* __restrict__ master, float* __restrict__ m, float* __restrict__ v,
                 const void* __restrict__ grad, int grad_fp32, __nv_bfloat16* __restrict__ pbf,
                 long long n, float lr, float b1, float b2, float eps, float wd, float c1,
                 float c2, float gscale, const float* __restrict__ hyper) {
  if (hyper) { lr = hyper[0]; c1 = hyper[1]; c2 = hyper[2]; gscale *= hyper[4]; }
  const long long n4 = n >> 2;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += stride) {
    if (!NKB_IN_BOUNDS(4 * i + 3, n)) continue;
    float4 p = reinterpret_cast<float4*>(master)[i];
    float4 mm = reinterpret_cast<float4*>(m)[i];
    float4 vv = reinterpret_cast<float4*>(v)[i];
    float g[4];
    if (grad_fp32) {
      float4 t = reinterpret_cast<const float4*>(grad)[i];
      g[0] = t.x; g[1] = t.y; g[2] = t.z; g[3] = t.w;
    } else {
      uint2 t = reinterpret_cast<const uint2*>(grad)[i];
      float2 a = unpack_bf16x2(t.x), b = unpack_bf16x2(t.y);
      g[0] = a.x; g[1] = a.y; g[2] = b.x; g[3] = b.y;
    }
    float pa[4] = {p.x, p.y, p.z, p.w}, ma[4] = {mm.x, mm.y, mm.z, mm.w},
          va[4] = {vv.x, vv.y, vv.z, vv.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float gj = g[j] * gscale;
      ma[j] = b1 * ma[j] + (1.f - b1) * gj;
      va[j] = b2 * va[j] + (1.f - b2) * gj * gj;
      float upd = (ma[j] * c1) / (sqrtf(va[j] * c2) + eps);
      pa[j] = pa[j] - lr * (upd + wd * pa[j]);
    }
    reinterpret_cast<float4*>(master)[i] = make_float4(pa[0], pa[1], pa[2], pa[3]);
    reinterpret_cast<float4*>(m)[i] = make_float4(ma[0], ma[1], ma[2], ma[3]);
    reinterpret_cast<float4*>(v)[i] = make_float4(va[0], va[1], va[2], va[3]);
    if (pbf)
      reinterpret_cast<uint2*>(pbf)[i] =
          make_uint2(pack_bf16x2(pa[0], pa[1]), pack_bf16x2(pa[2], pa[3]));
  }
  // tail (n % 4)
  for (long long i = (n4 << 2) + (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += stride) {
    float gj = load_as_float(grad, i, grad_fp32) * gscale;
    float mj = b1 * m[i] + (1.f - b1) * gj;
    float vj = b2 * v[i] + (1.f - b2) * gj * gj;
    float pj = master[i];
    pj = pj - lr * ((mj * c1) / (sqrtf(vj * c2) + eps) + wd * pj);
    m[i] = mj; v[i] = vj; master[i] = pj;
    if (pbf) pbf[i] = __float2bfloat16(pj);
  }
}

__global__ void __launch_bounds__(256)
sgd_flat_kernel(float* __restrict__ master, float* __restrict__ mom, const void* __restrict__ grad,
                int grad_fp32, __nv_bfloat16* __restrict__ pbf, long long n, float lr, float mu,
                float wd, float gscale, int first_step, const float* __restrict__ hyper) {
  if (hyper) { lr = hyper[0]; gscale *= hyper[4]; }
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    float p = master[i];
    float g = load_as_float(grad, i, grad_fp32) * gscale + wd * p;
    if (mom) {
      float b = first_step ? g : (mu * mom[i] + g);
      mom[i] = b;
      g = b;
    }
    p -= lr * g;
    master[i] = p;
    if (pbf) pbf[i] = __float2bfloat16(p);
  }
}

__device__ __forceinline__ uint32_t quant_code(float a, float thr, float& resid) {
  if (a >= thr) { resid = a - thr; return 1u; }
  if (a <= -thr) { resid = a + thr; return 2u; }
  resid = a;
  return 0u;
}
__device__ __forceinline__ float dequant_code(uint32_t code, float thr) {
  return code == 1u ? thr : (code == 2u ? -thr : 0.f);
}

// One thread packs one word = 16 consecutive elements.
__global__ void __launch_bounds__(256)
quant2_flat_kernel(const void* __restrict__ g, int g_fp32, float* __restrict__ residual,
                   uint32_t* __restrict__ codes, long long n, float thr) {
  const long long nwords = (n + 15) >> 4;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long w = (long long)blockIdx.x * blockDim.x + threadIdx.x; w < nwords; w += stride) {
    const long long base = w << 4;
    uint32_t word = 0;
    if (base + 16 <= n) {
      float a[16];
      if (g_fp32) {
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          float4 t = reinterpret_cast<const float4*>(static_cast<const float*>(g) + base)[q];
          a[4 * q] = t.x; a[4 * q + 1] = t.y; a[4 * q + 2] = t.z; a[4 * q + 3] = t.w;
        }
      } else {
#pragma unroll
        for (int q = 0; q < 2; ++q) {
          uint4 t = reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(g) + base)[q];
          uint32_t u[4] = {t.x, t.y, t.z, t.w};
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            float2 f = unpack_bf16x2(u[j]);
            a[8 * q + 2 * j] = f.x; a[8 * q + 2 * j + 1] = f.y;
          }
        }
      }
      float4* rp = reinterpret_cast<float4*>(residual + base);
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        float4 r = rp[q];
        float rr[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          float res;
          uint32_t c = quant_code(a[4 * q + j] + rr[j], thr, res);
          word |= c << (2 * (4 * q + j));
          rr[j] = res;
        }
        rp[q] = make_float4(rr[0], rr[1], rr[2], rr[3]);
      }
    } else {
      for (int i = 0; i < 16 && base + i < n; ++i) {
        float res;
        uint32_t c = quant_code(load_as_float(g, base + i, g_fp32) + residual[base + i], thr, res);
        word |= c << (2 * i);
        residual[base + i] = res;
      }
    }
    codes[w] = word;
  }
}

__global__ void __launch_bounds__(256)
dequant2_flat_kernel(const uint32_t* __restrict__ codes, void* __restrict__ out, int out_fp32,
                     long long n, float thr, float scale, int accumulate) {
  const long long nwords = (n + 15) >> 4;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long w = (long long)blockIdx.x * blockDim.x + threadIdx.x; w < nwords; w += stride) {
    const uint32_t word = codes[w];
    const long long base = w << 4;
    for (int i = 0; i < 16 && base + i < n; ++i) {
      float v = dequant_code((word >> (2 * i)) & 3u, thr) * scale;
      if (out_fp32) {
        float* o = static_cast<float*>(out) + base + i;
        *o = accumulate ? (*o + v) : v;
      } else {
        __nv_bfloat16* o = static_cast<__nv_bfloat16*>(out) + base + i;
        *o = __float2bfloat16(accumulate ? (__bfloat162float(*o) + v) : v);
      }
    }
  }
}

// Matrix packing (16 rows of one column -> one word); consecutive threads take
// consecutive columns so every row read is coalesced.
__global__ void __launch_bounds__(256)
quant2_matrix_kernel(const float* __restrict__ A, uint32_t* __restrict__ codes,
                     float* __restrict__ R, int n, int ncol, float thr) {
  const long long nwords = (long long)((n + 15) / 16) * ncol;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long w = (long long)blockIdx.x * blockDim.x + threadIdx.x; w < nwords; w += stride) {
    const int x = (int)(w / ncol), y = (int)(w % ncol);
    uint32_t word = 0;
    for (int i = 0; i < 16; ++i) {
      const int r = 16 * x + i;
      if (r >= n) break;
      float res;
      uint32_t c = quant_code(A[(long long)r * ncol + y], thr, res);
      word |= c << (2 * i);
      if (R) R[(long long)r * ncol + y] = res;
    }
    codes[w] = word;
  }
}
__global__ void __launch_bounds__(256)
dequant2_matrix_kernel(float* __restrict__ A, const uint32_t* __restrict__ codes, int n, int ncol,
                       float thr) {
  const long long nwords = (long long)((n + 15) / 16) * ncol;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long w = (long long)blockIdx.x * blockDim.x + threadIdx.x; w < nwords; w += stride) {
    const int x = (int)(w / ncol), y = (int)(w % ncol);
    const uint32_t word = codes[w];
    for (int i = 0; i < 16; ++i) {
      const int r = 16 * x + i;
      if (r >= n) break;
      A[(long long)r * ncol + y] = dequant_code((word >> (2 * i)) & 3u, thr);
    }
  }
}

__global__ void __launch_bounds__(256)
scale_cast_kernel(const void* __restrict__ src, int src_fp32, void* __restrict__ dst, int dst_fp32,
                  long long n, float scale, int accumulate) {
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    float v = load_as_float(src, i, src_fp32) * scale;
    if (dst_fp32) {
      float* o = static_cast<float*>(dst) + i;
      *o = accumulate ? (*o + v) : v;
    } else {
      __nv_bfloat16* o = static_cast<__nv_bfloat16*>(dst) + i;
      *o = __float2bfloat16(accumulate ? (__bfloat162float(*o) + v) : v);
    }
  }
}

__global__ void __launch_bounds__(256)
sumsq_kernel(const void* __restrict__ src, int src_fp32, long long n, float* __restrict__ out) {
  __shared__ float sh[8];
  float acc = 0.f;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    float v = load_as_float(src, i, src_fp32);
    acc += v * v;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x < 8) {
    acc = sh[threadIdx.x];
#pragma unroll
    for (int o = 4; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffu, acc, o);
    if (threadIdx.x == 0) atomicAdd(out, acc);
  }
}

static int grid_for(long long work_items) {
  long long b = (work_items + 255) / 256;
  const long long cap = 148 * 8;
  if (b > cap) b = cap;
  if (b < 1) b = 1;
  return (int)b;
}

// hyper[4] = min(1, max_norm / (sqrt(sumsq) * gscale)): the multiplier that clips the global
// gradient norm; applied inside the optimizer kernels.
__global__ void clip_coef_kernel(float* hyper, const float* sumsq, float max_norm, float gscale) {
  if (threadIdx.x == 0 && blockIdx.x == 0) {
    const float nrm = sqrtf(sumsq[0]) * gscale;
    hyper[4] = fminf(1.f, max_norm / (nrm + 1e-6f));
    hyper[5] = nrm;
  }
}

// Advances the optimizer's per-step scalars on the device: hyper = {lr, c1, c2, t}.
// t += 1; c1 = 1 / (1 - beta1^t); c2 = 1 / (1 - beta2^t).  One thread.  Keeping the step
// count on the device makes the values a function of how many steps the stream has run,
// not of when the host last rewrote a staging buffer (the host may enqueue many steps, or
// replay a CUDA graph, far ahead of the device).
__global__ void hyper_advance_kernel(float* hyper, float beta1, float beta2) {
  if (threadIdx.x == 0 && blockIdx.x == 0) {
    const float t = hyper[3] + 1.f;
    hyper[3] = t;
    // exact powers in double: 1 - beta^t loses its digits in fp32 for beta close to 1
    hyper[1] = (float)(1.0 / (1.0 - pow((double)beta1, (double)t)));
    hyper[2] = (float)(1.0 / (1.0 - pow((double)beta2, (double)t)));
  }
}

}  // namespace nkb

using namespace nkb;

extern "C" int nkb_clip_coef(float* hyper, const float* sumsq, float max_norm, float gscale,
                             void* stream) {
  clip_coef_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(hyper, sumsq, max_norm, gscale);
  return (int)cudaGetLastError();
}

extern "C" int nkb_hyper_advance(float* hyper, float beta1, float beta2, void* stream) {
  hyper_advance_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(hyper, beta1, beta2);
  return (int)cudaGetLastError();
}

extern "C" int nkb_adam_flat(float* master, float* m, float* v, const void* grad, int grad_fp32,
                             void* param_bf16, long long n, float lr, float beta1, float beta2,
                             float eps, float weight_decay, float bias_c1, float bias_c2,
                             float grad_scale, const float* hyper_dev, void* stream) {
  if (n <= 0) return 0;
  // 16-byte accesses need aligned bases
  if ((reinterpret_cast<uintptr_t>(master) | reinterpret_cast<uintptr_t>(m) |
       reinterpret_cast<uintptr_t>(v)) & 15)
    return -3;
  if (reinterpret_cast<uintptr_t>(grad) & (grad_fp32 ? 15 : 7)) return -3;
  if (param_bf16 && (reinterpret_cast<uintptr_t>(param_bf16) & 7)) return -3;
  adam_flat_kernel<<<grid_for(n / 4 + 1), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      master, m, v, grad, grad_fp32, static_cast<__nv_bfloat16*>(param_bf16), n, lr, beta1, beta2,
      eps, weight_decay, bias_c1, bias_c2, grad_scale, hyper_dev);
  return (int)cudaGetLastError();
}

extern "C" int nkb_sgd_flat(float* master, float* mom, const void* grad, int grad_fp32,
                            void* param_bf16, long long n, float lr, float momentum,
                            float weight_decay, float grad_scale, int first_step,
                            const float* hyper_dev, void* stream) {
  if (n <= 0) return 0;
  sgd_flat_kernel<<<grid_for(n), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      master, mom, grad, grad_fp32, static_cast<__nv_bfloat16*>(param_bf16), n, lr, momentum,
      weight_decay, grad_scale, first_step, hyper_dev);
  return (int)cudaGetLastError();
}

extern "C" int nkb_quant2_flat(const void* g, int g_fp32, float* residual, uint32_t* codes,
                               long long n, float thr, void* stream) {
  if (n <= 0) return 0;
  if ((reinterpret_cast<uintptr_t>(g) | reinterpret_cast<uintptr_t>(residual)) & 15) return -3;
  quant2_flat_kernel<<<grid_for((n + 15) / 16), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      g, g_fp32, residual, codes, n, thr);
  return (int)cudaGetLastError();
}
extern "C" int nkb_dequant2_flat(const uint32_t* codes, void* out, int out_fp32, long long n,
                                 float thr, float scale, int accumulate, void* stream) {
  if (n <= 0) return 0;
  dequant2_flat_kernel<<<grid_for((n + 15) / 16), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      codes, out, out_fp32, n, thr, scale, accumulate);
  return (int)cudaGetLastError();
}
extern "C" int nkb_quant2_matrix(const float* A, uint32_t* codes, float* R, int n, int ncol,
                                 float thr, void* stream) {
  if (n <= 0 || ncol <= 0) return 0;
  quant2_matrix_kernel<<<grid_for((long long)((n + 15) / 16) * ncol), 256, 0,
                         static_cast<cudaStream_t>(stream)>>>(A, codes, R, n, ncol, thr);
  return (int)cudaGetLastError();
}
extern "C" int nkb_dequant2_matrix(float* A, const uint32_t* codes, int n, int ncol, float thr,
                                   void* stream) {
  if (n <= 0 || ncol <= 0) return 0;
  dequant2_matrix_kernel<<<grid_for((long long)((n + 15) / 16) * ncol), 256, 0,
                           static_cast<cudaStream_t>(stream)>>>(A, codes, n, ncol, thr);
  return (int)cudaGetLastError();
}
extern "C" int nkb_scale_cast(const void* src, int src_fp32, void* dst, int dst_fp32, long long n,
                              float scale, int accumulate, void* stream) {
  if (n <= 0) return 0;
  scale_cast_kernel<<<grid_for(n), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      src, src_fp32, dst, dst_fp32, n, scale, accumulate);
  return (int)cudaGetLastError();
}
extern "C" int nkb_sumsq(const void* src, int src_fp32, long long n, float* out_accum,
                         void* stream) {
  if (n <= 0) return 0;
  sumsq_kernel<<<grid_for(n), 256, 0, static_cast<cudaStream_t>(stream)>>>(src, src_fp32, n,
                                                                          out_accum);
  return (int)cudaGetLastError();
}

extern "C" int nkb_num_sms(void) {
  int dev = 0, n = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return 0;
  cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
  return n;
}
extern "C" const char* nkb_build_info(void) {
  return "necklace_b200 native library, sm_100a, built " __DATE__ " " __TIME__;
}

NKB_DEFINE_BOUNDS_GETTER(optim)
