// Convolution support kernels for channels-last (NHWC) bf16 activations, batch
// normalisation (training mode) fused with ReLU and the residual add, and pooling.
//
// A convolution is a GEMM on the tcgen05 kernel of gemm_sm100.cu:
//   1x1 stride 1      activations [N*H*W, Cin] are the A operand as they are;
//   everything else   `im2col` gathers the receptive fields into col [N*Ho*Wo, KH*KW*Cin]
//                     (K index = (kh*KW + kw)*Cin + c, zero for padding), the weight is stored
//                     [Cout, KH*KW*Cin]; the data gradient is GEMM + `col2im` (written as a
//                     gather over the taps that touch an input pixel: no atomics, deterministic),
//                     the weight gradient is a GEMM over a recomputed col.
// The reference trains CNNs through torch's cuDNN convolutions
// (examples/dp/mnist/pytorch/main.py); these kernels take their place for the ResNet-50
// configuration.
#include "ptx.cuh"
#include "nkb_api.h"

namespace nkb {

static int conv_grid(long long work, int threads) {
  long long b = (work + threads - 1) / threads;
  const long long cap = 148LL * 16;
  if (b > cap) b = cap;
  if (b < 1) b = 1;
  return (int)b;
}

struct ConvGeom {
  int N, H, W, C, KH, KW, stride, pad, Ho, Wo, Kpad;
};

// VEC = 8: C % 8 == 0, 16-byte accesses; VEC = 1: any C.
template <int VEC>
__global__ void __launch_bounds__(256)
im2col_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ col, ConvGeom g) {
  const long long M = (long long)g.N * g.Ho * g.Wo;
  const int kchunks = g.Kpad / VEC;
  const int Kreal = g.KH * g.KW * g.C;
  const long long total = M * kchunks;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += stride) {
    const long long m = idx / kchunks;
    const int k = (int)(idx % kchunks) * VEC;
    const int wo = (int)(m % g.Wo);
    const long long t = m / g.Wo;
    const int ho = (int)(t % g.Ho);
    const int n = (int)(t / g.Ho);
    bool ok = k < Kreal;
    long long src = 0;
    if (ok) {
      const int tap = k / g.C, c = k % g.C;
      const int kh = tap / g.KW, kw = tap % g.KW;
      const int h = ho * g.stride - g.pad + kh, w = wo * g.stride - g.pad + kw;
      ok = h >= 0 && h < g.H && w >= 0 && w < g.W;
      src = (((long long)n * g.H + h) * g.W + w) * g.C + c;
    }
    const long long x_elems = (long long)g.N * g.H * g.W * g.C;
    if (ok && !NKB_IN_BOUNDS(src + VEC - 1, x_elems)) ok = false;
    if (!NKB_IN_BOUNDS(m * g.Kpad + k + VEC - 1, M * g.Kpad)) continue;
    if (VEC == 8) {
      uint4 v = make_uint4(0, 0, 0, 0);
      if (ok) v = *reinterpret_cast<const uint4*>(x + src);
      *reinterpret_cast<uint4*>(col + m * g.Kpad + k) = v;
    } else {
      col[m * g.Kpad + k] = ok ? x[src] : __float2bfloat16(0.f);
    }
  }
}

// Channel counts that are not a multiple of 8 (the 3-channel stem): one thread builds 8
// consecutive K entries (each with its own tap / channel, scalar 2-byte loads that hit the
// small, heavily reused input in cache) and writes them with one 16-byte store.
__global__ void __launch_bounds__(256)
im2col_gather8_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ col,
                      ConvGeom g) {
  const long long M = (long long)g.N * g.Ho * g.Wo;
  const int kchunks = g.Kpad / 8;
  const int Kreal = g.KH * g.KW * g.C;
  const long long total = M * kchunks;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += stride) {
    const long long m = idx / kchunks;
    const int k0 = (int)(idx % kchunks) * 8;
    const int wo = (int)(m % g.Wo);
    const long long t = m / g.Wo;
    const int ho = (int)(t % g.Ho);
    const int n = (int)(t / g.Ho);
    const int h0 = ho * g.stride - g.pad, w0 = wo * g.stride - g.pad;
    unsigned short v[8];
    int tap = k0 / g.C, c = k0 % g.C;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      unsigned short e = 0;
      if (k0 + j < Kreal) {
        const int kh = tap / g.KW, kw = tap % g.KW;
        const int h = h0 + kh, w = w0 + kw;
        if (h >= 0 && h < g.H && w >= 0 && w < g.W) {
          const long long src = (((long long)n * g.H + h) * g.W + w) * g.C + c;
          if (NKB_IN_BOUNDS(src, (long long)g.N * g.H * g.W * g.C))
            e = reinterpret_cast<const unsigned short*>(x)[src];
        }
      }
      v[j] = e;
      if (++c == g.C) { c = 0; ++tap; }
    }
    if (!NKB_IN_BOUNDS(m * g.Kpad + k0 + 7, M * g.Kpad)) continue;
    *reinterpret_cast<uint4*>(col + m * g.Kpad + k0) =
        make_uint4(v[0] | ((uint32_t)v[1] << 16), v[2] | ((uint32_t)v[3] << 16),
                   v[4] | ((uint32_t)v[5] << 16), v[6] | ((uint32_t)v[7] << 16));
  }
}

// dx[n,h,w,c] = sum over taps (kh,kw) with (h + pad - kh) % stride == 0 (same for w) of
// dcol[(n, (h+pad-kh)/stride, (w+pad-kw)/stride), (kh*KW+kw)*C + c]
template <int VEC>
__global__ void __launch_bounds__(256)
col2im_kernel(const __nv_bfloat16* __restrict__ dcol, __nv_bfloat16* __restrict__ dx, ConvGeom g) {
  const int cchunks = g.C / VEC;
  const long long total = (long long)g.N * g.H * g.W * cchunks;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += stride) {
    const int c = (int)(idx % cchunks) * VEC;
    long long t = idx / cchunks;
    const int w = (int)(t % g.W);
    t /= g.W;
    const int h = (int)(t % g.H);
    const int n = (int)(t / g.H);
    float acc[VEC];
#pragma unroll
    for (int j = 0; j < VEC; ++j) acc[j] = 0.f;
    for (int kh = 0; kh < g.KH; ++kh) {
      const int hn = h + g.pad - kh;
      if (hn < 0 || hn % g.stride) continue;
      const int ho = hn / g.stride;
      if (ho >= g.Ho) continue;
      for (int kw = 0; kw < g.KW; ++kw) {
        const int wn = w + g.pad - kw;
        if (wn < 0 || wn % g.stride) continue;
        const int wo = wn / g.stride;
        if (wo >= g.Wo) continue;
        const long long src = (((long long)n * g.Ho + ho) * g.Wo + wo) * g.Kpad +
                              (long long)(kh * g.KW + kw) * g.C + c;
        if (!NKB_IN_BOUNDS(src + VEC - 1, (long long)g.N * g.Ho * g.Wo * g.Kpad)) continue;
        if (VEC == 8) {
          uint4 v = *reinterpret_cast<const uint4*>(dcol + src);
          uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            float2 f = unpack_bf16x2(u[j]);
            acc[2 * j] += f.x;
            acc[2 * j + 1] += f.y;
          }
        } else {
          acc[0] += __bfloat162float(dcol[src]);
        }
      }
    }
    const long long dst = (((long long)n * g.H + h) * g.W + w) * g.C + c;
    if (VEC == 8) {
      *reinterpret_cast<uint4*>(dx + dst) =
          make_uint4(pack_bf16x2(acc[0], acc[1]), pack_bf16x2(acc[2], acc[3]),
                     pack_bf16x2(acc[4], acc[5]), pack_bf16x2(acc[6], acc[7]));
    } else {
      dx[dst] = __float2bfloat16(acc[0]);
    }
  }
}

// ------------------------------------------------------------------ batch norm
// Per-channel sums over the rows of a [M, C] matrix (C % 8 == 0):
//   MODE 0: acc[0][c] += sum x,        acc[1][c] += sum x^2            (forward statistics)
//   MODE 1: acc[0][c] += sum dy',      acc[1][c] += sum dy' * xhat     (backward sums)
// with dy' = dy * (y > 0) when relu (y = the layer's output), xhat = (x - mean) * rstd.
// Threads: 8 channels each; a block covers `cx` channel chunks x `ry` row lanes.
template <int MODE>
__global__ void __launch_bounds__(256)
bn_sums_kernel(const __nv_bfloat16* __restrict__ a, const __nv_bfloat16* __restrict__ x,
               const __nv_bfloat16* __restrict__ y, const float* __restrict__ stats,
               float* __restrict__ acc, long long M, int C, int cx, int relu) {
  __shared__ float sh[2][256][8 + 1];
  const int ry = 256 / cx;
  const int tx = threadIdx.x % cx, ty = threadIdx.x / cx;
  const int c = (blockIdx.x * cx + tx) * 8;
  float s0[8], s1[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) s0[j] = s1[j] = 0.f;
  if (c < C && ty < ry) {
    float mean[8], rstd[8];
    if (MODE == 1) {
#pragma unroll
      for (int j = 0; j < 8; ++j) { mean[j] = stats[c + j]; rstd[j] = stats[C + c + j]; }
    }
    for (long long r = (long long)blockIdx.y * ry + ty; r < M; r += (long long)gridDim.y * ry) {
      uint4 va = *reinterpret_cast<const uint4*>(a + r * C + c);
      uint32_t ua[4] = {va.x, va.y, va.z, va.w};
      float fa[8];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float2 f = unpack_bf16x2(ua[j]);
        fa[2 * j] = f.x; fa[2 * j + 1] = f.y;
      }
      if (MODE == 0) {
#pragma unroll
        for (int j = 0; j < 8; ++j) { s0[j] += fa[j]; s1[j] += fa[j] * fa[j]; }
      } else {
        uint4 vx = *reinterpret_cast<const uint4*>(x + r * C + c);
        uint32_t ux[4] = {vx.x, vx.y, vx.z, vx.w};
        float fx[8];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          float2 f = unpack_bf16x2(ux[j]);
          fx[2 * j] = f.x; fx[2 * j + 1] = f.y;
        }
        if (relu) {
          uint4 vy = *reinterpret_cast<const uint4*>(y + r * C + c);
          uint32_t uy[4] = {vy.x, vy.y, vy.z, vy.w};
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            float2 f = unpack_bf16x2(uy[j]);
            if (!(f.x > 0.f)) fa[2 * j] = 0.f;
            if (!(f.y > 0.f)) fa[2 * j + 1] = 0.f;
          }
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          s0[j] += fa[j];
          s1[j] += fa[j] * (fx[j] - mean[j]) * rstd[j];
        }
      }
    }
  }
#pragma unroll
  for (int j = 0; j < 8; ++j) { sh[0][threadIdx.x][j] = s0[j]; sh[1][threadIdx.x][j] = s1[j]; }
  __syncthreads();
  // the first cx*8 threads each own one channel of the strip and add up the row lanes
  if (threadIdx.x < cx * 8) {
    const int chunk = threadIdx.x / 8, j = threadIdx.x % 8;
    const int cc = (blockIdx.x * cx + chunk) * 8 + j;
    if (cc < C) {
      float t0 = 0.f, t1 = 0.f;
      for (int l = 0; l < ry; ++l) {
        t0 += sh[0][l * cx + chunk][j];
        t1 += sh[1][l * cx + chunk][j];
      }
      atomicAdd(acc + cc, t0);
      atomicAdd(acc + C + cc, t1);
    }
  }
}

// stats[0][c] = mean, stats[1][c] = rstd from the forward sums; running statistics updated
// (momentum form of torch.nn.BatchNorm2d, unbiased variance); the accumulator is re-zeroed.
__global__ void bn_finalize_kernel(float* __restrict__ acc, float* __restrict__ stats,
                                   float* __restrict__ run_mean, float* __restrict__ run_var,
                                   long long M, int C, float eps, float momentum) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  const float inv = 1.f / (float)M;
  const float mean = acc[c] * inv;
  float var = acc[C + c] * inv - mean * mean;
  var = fmaxf(var, 0.f);
  stats[c] = mean;
  stats[C + c] = rsqrtf(var + eps);
  if (run_mean) {
    const float unb = M > 1 ? var * (float)M / (float)(M - 1) : var;
    run_mean[c] = (1.f - momentum) * run_mean[c] + momentum * mean;
    run_var[c] = (1.f - momentum) * run_var[c] + momentum * unb;
  }
  acc[c] = 0.f;
  acc[C + c] = 0.f;
}

// y = act((x - mean) * rstd * gamma + beta (+ res)).  Thread layout as in bn_sums_kernel: a
// thread owns 8 fixed channels (its per-channel constants stay in registers) and walks rows.
__global__ void __launch_bounds__(256)
bn_apply_kernel(const __nv_bfloat16* __restrict__ x, const float* __restrict__ stats,
                const __nv_bfloat16* __restrict__ gamma, const __nv_bfloat16* __restrict__ beta,
                const __nv_bfloat16* __restrict__ res, __nv_bfloat16* __restrict__ y, long long M,
                int C, int cx, int relu) {
  const int ry = 256 / cx;
  const int tx = threadIdx.x % cx, ty = threadIdx.x / cx;
  const int c = (blockIdx.x * cx + tx) * 8;
  if (c >= C) return;
  float sc[8], sh[8];
  {
    uint4 vg = *reinterpret_cast<const uint4*>(gamma + c);
    uint4 vb = *reinterpret_cast<const uint4*>(beta + c);
    uint32_t ug[4] = {vg.x, vg.y, vg.z, vg.w}, ub[4] = {vb.x, vb.y, vb.z, vb.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float2 fg = unpack_bf16x2(ug[j]), fb = unpack_bf16x2(ub[j]);
      sc[2 * j] = stats[C + c + 2 * j] * fg.x;
      sc[2 * j + 1] = stats[C + c + 2 * j + 1] * fg.y;
      sh[2 * j] = fb.x - stats[c + 2 * j] * sc[2 * j];
      sh[2 * j + 1] = fb.y - stats[c + 2 * j + 1] * sc[2 * j + 1];
    }
  }
  for (long long r = (long long)blockIdx.y * ry + ty; r < M; r += (long long)gridDim.y * ry) {
    const long long off = r * C + c;
    uint4 vx = *reinterpret_cast<const uint4*>(x + off);
    uint32_t ux[4] = {vx.x, vx.y, vx.z, vx.w};
    uint32_t ur[4] = {0, 0, 0, 0};
    if (res) {
      uint4 vr = *reinterpret_cast<const uint4*>(res + off);
      ur[0] = vr.x; ur[1] = vr.y; ur[2] = vr.z; ur[3] = vr.w;
    }
    uint32_t o[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float2 fx = unpack_bf16x2(ux[j]), fr = unpack_bf16x2(ur[j]);
      float a = fx.x * sc[2 * j] + sh[2 * j] + fr.x;
      float b = fx.y * sc[2 * j + 1] + sh[2 * j + 1] + fr.y;
      if (relu) { a = fmaxf(a, 0.f); b = fmaxf(b, 0.f); }
      o[j] = pack_bf16x2(a, b);
    }
    *reinterpret_cast<uint4*>(y + off) = make_uint4(o[0], o[1], o[2], o[3]);
  }
}

// dx = gamma * rstd * (dy' - s0/M - xhat * s1/M);  dres = dy' (optional);
// sums = [2][C] from bn_sums_kernel<1>.  Same thread layout.
__global__ void __launch_bounds__(256)
bn_bwd_apply_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                    const __nv_bfloat16* __restrict__ y, const float* __restrict__ stats,
                    const float* __restrict__ sums, const __nv_bfloat16* __restrict__ gamma,
                    __nv_bfloat16* __restrict__ dx, __nv_bfloat16* __restrict__ dres, long long M,
                    int C, int cx, int relu) {
  const int ry = 256 / cx;
  const int tx = threadIdx.x % cx, ty = threadIdx.x / cx;
  const int c = (blockIdx.x * cx + tx) * 8;
  if (c >= C) return;
  const float invM = 1.f / (float)M;
  // dx = k1 * dy' + k2 * x + k3 with k1 = gamma rstd, k2 = -k1 rstd s1/M,
  // k3 = -k1 (s0/M - mean rstd s1/M)
  float k1[8], k2[8], k3[8];
  {
    uint4 vg = *reinterpret_cast<const uint4*>(gamma + c);
    uint32_t ug[4] = {vg.x, vg.y, vg.z, vg.w};
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float2 fg = unpack_bf16x2(ug[j >> 1]);
      const float g = (j & 1) ? fg.y : fg.x;
      const float mean = stats[c + j], rstd = stats[C + c + j];
      const float a0 = sums[c + j] * invM, a1 = sums[C + c + j] * invM;
      k1[j] = g * rstd;
      k2[j] = -k1[j] * rstd * a1;
      k3[j] = -k1[j] * (a0 - mean * rstd * a1);
    }
  }
  for (long long r = (long long)blockIdx.y * ry + ty; r < M; r += (long long)gridDim.y * ry) {
    const long long off = r * C + c;
    uint4 vd = *reinterpret_cast<const uint4*>(dy + off);
    uint4 vx = *reinterpret_cast<const uint4*>(x + off);
    uint32_t ud[4] = {vd.x, vd.y, vd.z, vd.w}, ux[4] = {vx.x, vx.y, vx.z, vx.w};
    uint32_t uy[4] = {0, 0, 0, 0};
    if (relu) {
      uint4 vy = *reinterpret_cast<const uint4*>(y + off);
      uy[0] = vy.x; uy[1] = vy.y; uy[2] = vy.z; uy[3] = vy.w;
    }
    uint32_t o[4], rr[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float2 fd = unpack_bf16x2(ud[j]), fx = unpack_bf16x2(ux[j]);
      if (relu) {
        float2 fy = unpack_bf16x2(uy[j]);
        if (!(fy.x > 0.f)) fd.x = 0.f;
        if (!(fy.y > 0.f)) fd.y = 0.f;
      }
      o[j] = pack_bf16x2(k1[2 * j] * fd.x + k2[2 * j] * fx.x + k3[2 * j],
                         k1[2 * j + 1] * fd.y + k2[2 * j + 1] * fx.y + k3[2 * j + 1]);
      rr[j] = pack_bf16x2(fd.x, fd.y);
    }
    *reinterpret_cast<uint4*>(dx + off) = make_uint4(o[0], o[1], o[2], o[3]);
    if (dres) *reinterpret_cast<uint4*>(dres + off) = make_uint4(rr[0], rr[1], rr[2], rr[3]);
  }
}

// dgamma / dbeta (bf16, written or accumulated) from the backward sums; sums re-zeroed.
__global__ void bn_param_grad_kernel(float* __restrict__ sums, __nv_bfloat16* __restrict__ dgamma,
                                     __nv_bfloat16* __restrict__ dbeta, int C, int acc_g,
                                     int acc_b) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  float g = sums[C + c], b = sums[c];
  if (dgamma) {
    if (acc_g) g += __bfloat162float(dgamma[c]);
    dgamma[c] = __float2bfloat16(g);
  }
  if (dbeta) {
    if (acc_b) b += __bfloat162float(dbeta[c]);
    dbeta[c] = __float2bfloat16(b);
  }
  sums[c] = 0.f;
  sums[C + c] = 0.f;
}

// --------------------------------------------------------------------- pooling
// 3x3 / stride 2 / pad 1 max pooling, NHWC, C % 8 == 0; idx = winning tap (0..8) per element.
__global__ void __launch_bounds__(256)
maxpool_fwd_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ y,
                   uint8_t* __restrict__ idx, int N, int H, int W, int C, int Ho, int Wo) {
  const int cch = C / 8;
  const long long total = (long long)N * Ho * Wo * cch;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
    const int c = (int)(i % cch) * 8;
    long long t = i / cch;
    const int wo = (int)(t % Wo);
    t /= Wo;
    const int ho = (int)(t % Ho);
    const int n = (int)(t / Ho);
    float best[8];
    int arg[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) { best[j] = -INFINITY; arg[j] = 0; }
    for (int kh = 0; kh < 3; ++kh) {
      const int h = ho * 2 - 1 + kh;
      if (h < 0 || h >= H) continue;
      for (int kw = 0; kw < 3; ++kw) {
        const int w = wo * 2 - 1 + kw;
        if (w < 0 || w >= W) continue;
        const long long src = (((long long)n * H + h) * W + w) * C + c;
        if (!NKB_IN_BOUNDS(src + 7, (long long)N * H * W * C)) continue;
        uint4 v = *reinterpret_cast<const uint4*>(x + src);
        uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          float2 f = unpack_bf16x2(u[j]);
          if (f.x > best[2 * j]) { best[2 * j] = f.x; arg[2 * j] = kh * 3 + kw; }
          if (f.y > best[2 * j + 1]) { best[2 * j + 1] = f.y; arg[2 * j + 1] = kh * 3 + kw; }
        }
      }
    }
    const long long dst = (((long long)n * Ho + ho) * Wo + wo) * C + c;
    *reinterpret_cast<uint4*>(y + dst) =
        make_uint4(pack_bf16x2(best[0], best[1]), pack_bf16x2(best[2], best[3]),
                   pack_bf16x2(best[4], best[5]), pack_bf16x2(best[6], best[7]));
    uint32_t lo = arg[0] | (arg[1] << 8) | (arg[2] << 16) | (arg[3] << 24);
    uint32_t hi = arg[4] | (arg[5] << 8) | (arg[6] << 16) | (arg[7] << 24);
    *reinterpret_cast<uint2*>(idx + dst) = make_uint2(lo, hi);
  }
}

__global__ void __launch_bounds__(256)
maxpool_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const uint8_t* __restrict__ idx,
                   __nv_bfloat16* __restrict__ dx, int N, int H, int W, int C, int Ho, int Wo) {
  const int cch = C / 8;
  const long long total = (long long)N * H * W * cch;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
    const int c = (int)(i % cch) * 8;
    long long t = i / cch;
    const int w = (int)(t % W);
    t /= W;
    const int h = (int)(t % H);
    const int n = (int)(t / H);
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
    for (int kh = 0; kh < 3; ++kh) {
      const int hn = h + 1 - kh;
      if (hn < 0 || (hn & 1)) continue;
      const int ho = hn >> 1;
      if (ho >= Ho) continue;
      for (int kw = 0; kw < 3; ++kw) {
        const int wn = w + 1 - kw;
        if (wn < 0 || (wn & 1)) continue;
        const int wo = wn >> 1;
        if (wo >= Wo) continue;
        const long long src = (((long long)n * Ho + ho) * Wo + wo) * C + c;
        if (!NKB_IN_BOUNDS(src + 7, (long long)N * Ho * Wo * C)) continue;
        uint2 iv = *reinterpret_cast<const uint2*>(idx + src);
        uint4 v = *reinterpret_cast<const uint4*>(dy + src);
        uint32_t u[4] = {v.x, v.y, v.z, v.w};
        const int tap = kh * 3 + kw;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          float2 f = unpack_bf16x2(u[j]);
          const uint32_t word = (2 * j < 4) ? iv.x : iv.y;
          const int a0 = (word >> (8 * ((2 * j) & 3))) & 0xff;
          const int a1 = (word >> (8 * ((2 * j + 1) & 3))) & 0xff;
          if (a0 == tap) acc[2 * j] += f.x;
          if (a1 == tap) acc[2 * j + 1] += f.y;
        }
      }
    }
    *reinterpret_cast<uint4*>(dx + (((long long)n * H + h) * W + w) * C + c) =
        make_uint4(pack_bf16x2(acc[0], acc[1]), pack_bf16x2(acc[2], acc[3]),
                   pack_bf16x2(acc[4], acc[5]), pack_bf16x2(acc[6], acc[7]));
  }
}

// Global average pooling over HW: x [N, HW, C] -> y [N, C]; backward spreads dy / HW.
__global__ void __launch_bounds__(256)
avgpool_fwd_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ y, int N,
                   int HW, int C) {
  const int cch = C / 8;
  const long long total = (long long)N * cch;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int c = (int)(i % cch) * 8;
    const int n = (int)(i / cch);
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
    for (int p = 0; p < HW; ++p) {
      uint4 v = *reinterpret_cast<const uint4*>(x + ((long long)n * HW + p) * C + c);
      uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float2 f = unpack_bf16x2(u[j]);
        acc[2 * j] += f.x;
        acc[2 * j + 1] += f.y;
      }
    }
    const float inv = 1.f / (float)HW;
    *reinterpret_cast<uint4*>(y + (long long)n * C + c) =
        make_uint4(pack_bf16x2(acc[0] * inv, acc[1] * inv), pack_bf16x2(acc[2] * inv, acc[3] * inv),
                   pack_bf16x2(acc[4] * inv, acc[5] * inv), pack_bf16x2(acc[6] * inv, acc[7] * inv));
  }
}

__global__ void __launch_bounds__(256)
avgpool_bwd_kernel(const __nv_bfloat16* __restrict__ dy, __nv_bfloat16* __restrict__ dx, int N,
                   int HW, int C) {
  const int cch = C / 8;
  const long long total = (long long)N * HW * cch;
  const float inv = 1.f / (float)HW;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int c = (int)(i % cch) * 8;
    const long long t = i / cch;
    const int n = (int)(t / HW);
    uint4 v = *reinterpret_cast<const uint4*>(dy + (long long)n * C + c);
    uint32_t u[4] = {v.x, v.y, v.z, v.w}, o[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float2 f = unpack_bf16x2(u[j]);
      o[j] = pack_bf16x2(f.x * inv, f.y * inv);
    }
    *reinterpret_cast<uint4*>(dx + t * C + c) = make_uint4(o[0], o[1], o[2], o[3]);
  }
}

}  // namespace nkb

using namespace nkb;

static ConvGeom geom(int N, int H, int W, int C, int KH, int KW, int stride, int pad, int Kpad) {
  ConvGeom g;
  g.N = N; g.H = H; g.W = W; g.C = C; g.KH = KH; g.KW = KW; g.stride = stride; g.pad = pad;
  g.Ho = (H + 2 * pad - KH) / stride + 1;
  g.Wo = (W + 2 * pad - KW) / stride + 1;
  g.Kpad = Kpad;
  return g;
}

extern "C" int nkb_im2col_nhwc(const void* x, void* col, int N, int H, int W, int C, int KH,
                               int KW, int stride, int pad, int Kpad, void* stream) {
  if (Kpad < KH * KW * C || (Kpad & 7)) return -3;
  ConvGeom g = geom(N, H, W, C, KH, KW, stride, pad, Kpad);
  if (g.Ho <= 0 || g.Wo <= 0) return -2;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const long long M = (long long)N * g.Ho * g.Wo;
  const bool vec = (C % 8 == 0) && !(reinterpret_cast<uintptr_t>(x) & 15) &&
                   !(reinterpret_cast<uintptr_t>(col) & 15);
  if (vec)
    im2col_kernel<8><<<conv_grid(M * (Kpad / 8), 256), 256, 0, s>>>(
        static_cast<const __nv_bfloat16*>(x), static_cast<__nv_bfloat16*>(col), g);
  else if (!(reinterpret_cast<uintptr_t>(col) & 15))
    im2col_gather8_kernel<<<conv_grid(M * (Kpad / 8), 256), 256, 0, s>>>(
        static_cast<const __nv_bfloat16*>(x), static_cast<__nv_bfloat16*>(col), g);
  else
    im2col_kernel<1><<<conv_grid(M * Kpad, 256), 256, 0, s>>>(
        static_cast<const __nv_bfloat16*>(x), static_cast<__nv_bfloat16*>(col), g);
  return (int)cudaGetLastError();
}

extern "C" int nkb_col2im_nhwc(const void* dcol, void* dx, int N, int H, int W, int C, int KH,
                               int KW, int stride, int pad, int Kpad, void* stream) {
  if (Kpad < KH * KW * C || (Kpad & 7)) return -3;
  ConvGeom g = geom(N, H, W, C, KH, KW, stride, pad, Kpad);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const bool vec = (C % 8 == 0) && !(reinterpret_cast<uintptr_t>(dx) & 15) &&
                   !(reinterpret_cast<uintptr_t>(dcol) & 15);
  const long long px = (long long)N * H * W;
  if (vec)
    col2im_kernel<8><<<conv_grid(px * (C / 8), 256), 256, 0, s>>>(
        static_cast<const __nv_bfloat16*>(dcol), static_cast<__nv_bfloat16*>(dx), g);
  else
    col2im_kernel<1><<<conv_grid(px * C, 256), 256, 0, s>>>(
        static_cast<const __nv_bfloat16*>(dcol), static_cast<__nv_bfloat16*>(dx), g);
  return (int)cudaGetLastError();
}

static void bn_sums_dims(long long M, int C, int& cx, dim3& grid) {
  const int chunks = C / 8;
  cx = chunks >= 32 ? 32 : (chunks >= 16 ? 16 : (chunks >= 8 ? 8 : (chunks >= 4 ? 4 :
       (chunks >= 2 ? 2 : 1))));
  const int gx = (chunks + cx - 1) / cx;
  const int ry = 256 / cx;
  long long gy = (148LL * 8) / gx;
  const long long need = (M + ry - 1) / ry;
  if (gy > need) gy = need;
  if (gy < 1) gy = 1;
  if (gy > 65535) gy = 65535;
  grid = dim3(gx, (unsigned)gy);
}

// Forward: batch statistics of x [M, C], then y = act(bn(x) (+ res)).  acc: fp32 [2][C], zero on
// entry, left zero.  stats out: fp32 [2][C] (mean, rstd).
extern "C" int nkb_bn_fwd(const void* x, const void* gamma, const void* beta, const void* res,
                          void* y, float* stats, float* acc, float* run_mean, float* run_var,
                          long long M, int C, float eps, float momentum, int relu, void* stream) {
  if (C % 8) return -3;
  if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y) |
       reinterpret_cast<uintptr_t>(gamma) | reinterpret_cast<uintptr_t>(beta)) & 15)
    return -3;
  if (res && (reinterpret_cast<uintptr_t>(res) & 15)) return -3;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  int cx;
  dim3 grid;
  bn_sums_dims(M, C, cx, grid);
  bn_sums_kernel<0><<<grid, 256, 0, s>>>(static_cast<const __nv_bfloat16*>(x), nullptr, nullptr,
                                         nullptr, acc, M, C, cx, 0);
  bn_finalize_kernel<<<(C + 127) / 128, 128, 0, s>>>(acc, stats, run_mean, run_var, M, C, eps,
                                                     momentum);
  bn_apply_kernel<<<grid, 256, 0, s>>>(
      static_cast<const __nv_bfloat16*>(x), stats, static_cast<const __nv_bfloat16*>(gamma),
      static_cast<const __nv_bfloat16*>(beta), static_cast<const __nv_bfloat16*>(res),
      static_cast<__nv_bfloat16*>(y), M, C, cx, relu);
  return (int)cudaGetLastError();
}

// Evaluation mode: y = act((x - mean) * rstd * gamma + beta (+ res)) with given stats [2][C].
extern "C" int nkb_bn_apply(const void* x, const float* stats, const void* gamma, const void* beta,
                            const void* res, void* y, long long M, int C, int relu, void* stream) {
  if (C % 8) return -3;
  int cx;
  dim3 grid;
  bn_sums_dims(M, C, cx, grid);
  bn_apply_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(x), stats, static_cast<const __nv_bfloat16*>(gamma),
      static_cast<const __nv_bfloat16*>(beta), static_cast<const __nv_bfloat16*>(res),
      static_cast<__nv_bfloat16*>(y), M, C, cx, relu);
  return (int)cudaGetLastError();
}

// Backward: dx (and dres = relu-masked dy when given), dgamma / dbeta written or accumulated.
extern "C" int nkb_bn_bwd(const void* dy, const void* x, const void* y, const float* stats,
                          const void* gamma, void* dx, void* dres, void* dgamma, void* dbeta,
                          int acc_g, int acc_b, float* acc, long long M, int C, int relu,
                          void* stream) {
  if (C % 8) return -3;
  if ((reinterpret_cast<uintptr_t>(dy) | reinterpret_cast<uintptr_t>(x) |
       reinterpret_cast<uintptr_t>(dx) | reinterpret_cast<uintptr_t>(gamma)) & 15)
    return -3;
  if (relu && (y == nullptr || (reinterpret_cast<uintptr_t>(y) & 15))) return -3;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  int cx;
  dim3 grid;
  bn_sums_dims(M, C, cx, grid);
  bn_sums_kernel<1><<<grid, 256, 0, s>>>(static_cast<const __nv_bfloat16*>(dy),
                                         static_cast<const __nv_bfloat16*>(x),
                                         static_cast<const __nv_bfloat16*>(y), stats, acc, M, C,
                                         cx, relu);
  bn_bwd_apply_kernel<<<grid, 256, 0, s>>>(
      static_cast<const __nv_bfloat16*>(dy), static_cast<const __nv_bfloat16*>(x),
      static_cast<const __nv_bfloat16*>(y), stats, acc, static_cast<const __nv_bfloat16*>(gamma),
      static_cast<__nv_bfloat16*>(dx), static_cast<__nv_bfloat16*>(dres), M, C, cx, relu);
  bn_param_grad_kernel<<<(C + 127) / 128, 128, 0, s>>>(acc, static_cast<__nv_bfloat16*>(dgamma),
                                                       static_cast<__nv_bfloat16*>(dbeta), C,
                                                       acc_g, acc_b);
  return (int)cudaGetLastError();
}

extern "C" int nkb_maxpool3x3s2_fwd(const void* x, void* y, void* idx, int N, int H, int W, int C,
                                    void* stream) {
  if (C % 8) return -3;
  const int Ho = (H + 2 - 3) / 2 + 1, Wo = (W + 2 - 3) / 2 + 1;
  maxpool_fwd_kernel<<<conv_grid((long long)N * Ho * Wo * (C / 8), 256), 256, 0,
                       static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(x), static_cast<__nv_bfloat16*>(y),
      static_cast<uint8_t*>(idx), N, H, W, C, Ho, Wo);
  return (int)cudaGetLastError();
}

extern "C" int nkb_maxpool3x3s2_bwd(const void* dy, const void* idx, void* dx, int N, int H, int W,
                                    int C, void* stream) {
  if (C % 8) return -3;
  const int Ho = (H + 2 - 3) / 2 + 1, Wo = (W + 2 - 3) / 2 + 1;
  maxpool_bwd_kernel<<<conv_grid((long long)N * H * W * (C / 8), 256), 256, 0,
                       static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(dy), static_cast<const uint8_t*>(idx),
      static_cast<__nv_bfloat16*>(dx), N, H, W, C, Ho, Wo);
  return (int)cudaGetLastError();
}

extern "C" int nkb_avgpool_fwd(const void* x, void* y, int N, int HW, int C, void* stream) {
  if (C % 8) return -3;
  avgpool_fwd_kernel<<<conv_grid((long long)N * (C / 8), 256), 256, 0,
                       static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(x), static_cast<__nv_bfloat16*>(y), N, HW, C);
  return (int)cudaGetLastError();
}

extern "C" int nkb_avgpool_bwd(const void* dy, void* dx, int N, int HW, int C, void* stream) {
  if (C % 8) return -3;
  avgpool_bwd_kernel<<<conv_grid((long long)N * HW * (C / 8), 256), 256, 0,
                       static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(dy), static_cast<__nv_bfloat16*>(dx), N, HW, C);
  return (int)cudaGetLastError();
}

NKB_DEFINE_BOUNDS_GETTER(conv)

#ifdef NKB_DEBUG_BOUNDS
// Exercises the reporting path of the debug build without touching memory: one failing
// check (index 5 of an extent of 4) is evaluated and nothing is accessed.
namespace nkb {
__global__ void bounds_selftest_kernel(int* sink) {
  if (NKB_IN_BOUNDS(5, 4)) *sink = 1;
}
}  // namespace nkb
extern "C" int nkb_debug_bounds_selftest(int* sink, void* stream) {
  nkb::bounds_selftest_kernel<<<1, 1, 0, static_cast<cudaStream_t>(stream)>>>(sink);
  return (int)cudaGetLastError();
}
#endif
