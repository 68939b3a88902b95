// Rotary position embedding (in place on the packed QKV buffer) and SwiGLU
// forward / backward, bf16 activations with fp32 math.  Memory-bound kernels:
// 16-byte accesses, one pass over the data.  The reference has neither op; they
// serve the Llama-style configurations.
#include "ptx.cuh"
#include "nkb_api.h"

namespace nkb {

// qkv: [T = B*S, 3*C] with C = H*D.  Rotates the q and k parts: for head h and
// i < D/2 the pair (x[i], x[i + D/2]) is rotated by angle pos * base^(-2i/D).
// dir = +1 forward, -1 backward (inverse rotation).  One thread handles 8
// consecutive i of one (token, head, q-or-k).
__global__ void __launch_bounds__(256)
rope_kernel(__nv_bfloat16* __restrict__ qkv, int T, int S, int H, int D, float base, float dir,
            int pos_offset) {
  const int half = D / 2;
  const int groups = half / 8;
  const long long total = (long long)T * 2 * H * groups;
  const int C = H * D;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const int gi = (int)(idx % groups);
    long long r = idx / groups;
    const int h = (int)(r % H);
    r /= H;
    const int which = (int)(r % 2);  // 0 = q, 1 = k
    const long long t = r / 2;
    const int pos = (int)(t % S) + pos_offset;
    __nv_bfloat16* p = qkv + t * 3LL * C + (long long)which * C + (long long)h * D + gi * 8;
    uint4 lo = *reinterpret_cast<uint4*>(p);
    uint4 hi = *reinterpret_cast<uint4*>(p + half);
    uint32_t l[4] = {lo.x, lo.y, lo.z, lo.w}, u[4] = {hi.x, hi.y, hi.z, hi.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float2 a = unpack_bf16x2(l[j]), b = unpack_bf16x2(u[j]);
      const int i0 = gi * 8 + 2 * j;
      float s0, c0, s1, c1;
      __sincosf(pos * __powf(base, -2.f * i0 / D), &s0, &c0);
      __sincosf(pos * __powf(base, -2.f * (i0 + 1) / D), &s1, &c1);
      s0 *= dir;
      s1 *= dir;
      l[j] = pack_bf16x2(a.x * c0 - b.x * s0, a.y * c1 - b.y * s1);
      u[j] = pack_bf16x2(b.x * c0 + a.x * s0, b.y * c1 + a.y * s1);
    }
    *reinterpret_cast<uint4*>(p) = make_uint4(l[0], l[1], l[2], l[3]);
    *reinterpret_cast<uint4*>(p + half) = make_uint4(u[0], u[1], u[2], u[3]);
  }
}

__device__ __forceinline__ float sigmoidf_(float x) { return 1.f / (1.f + __expf(-x)); }

// gu: [T, 2F] (gate | up); h: [T, F] = silu(gate) * up
__global__ void __launch_bounds__(256)
swiglu_fwd_kernel(const __nv_bfloat16* __restrict__ gu, __nv_bfloat16* __restrict__ h, long long T,
                  int F) {
  const int f8 = F / 8;
  const long long total = T * f8;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const long long t = idx / f8;
    const int c = (int)(idx % f8) * 8;
    uint4 g = ld_nc_v4(gu + t * 2LL * F + c);
    uint4 u = ld_nc_v4(gu + t * 2LL * F + F + c);
    uint32_t gw[4] = {g.x, g.y, g.z, g.w}, uw[4] = {u.x, u.y, u.z, u.w}, o[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float2 a = unpack_bf16x2(gw[j]), b = unpack_bf16x2(uw[j]);
      o[j] = pack_bf16x2(a.x * sigmoidf_(a.x) * b.x, a.y * sigmoidf_(a.y) * b.y);
    }
    *reinterpret_cast<uint4*>(h + t * (long long)F + c) = make_uint4(o[0], o[1], o[2], o[3]);
  }
}

// dgu[:, :F] = dh * up * silu'(gate) ; dgu[:, F:] = dh * silu(gate)
__global__ void __launch_bounds__(256)
swiglu_bwd_kernel(const __nv_bfloat16* __restrict__ gu, const __nv_bfloat16* __restrict__ dh,
                  __nv_bfloat16* __restrict__ dgu, long long T, int F) {
  const int f8 = F / 8;
  const long long total = T * f8;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const long long t = idx / f8;
    const int c = (int)(idx % f8) * 8;
    uint4 g = ld_nc_v4(gu + t * 2LL * F + c);
    uint4 u = ld_nc_v4(gu + t * 2LL * F + F + c);
    uint4 d = ld_nc_v4(dh + t * (long long)F + c);
    uint32_t gw[4] = {g.x, g.y, g.z, g.w}, uw[4] = {u.x, u.y, u.z, u.w},
             dw[4] = {d.x, d.y, d.z, d.w}, og[4], ou[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float2 a = unpack_bf16x2(gw[j]), b = unpack_bf16x2(uw[j]), e = unpack_bf16x2(dw[j]);
      float s0 = sigmoidf_(a.x), s1 = sigmoidf_(a.y);
      float silu0 = a.x * s0, silu1 = a.y * s1;
      float ds0 = s0 * (1.f + a.x * (1.f - s0)), ds1 = s1 * (1.f + a.y * (1.f - s1));
      og[j] = pack_bf16x2(e.x * b.x * ds0, e.y * b.y * ds1);
      ou[j] = pack_bf16x2(e.x * silu0, e.y * silu1);
    }
    *reinterpret_cast<uint4*>(dgu + t * 2LL * F + c) = make_uint4(og[0], og[1], og[2], og[3]);
    *reinterpret_cast<uint4*>(dgu + t * 2LL * F + F + c) = make_uint4(ou[0], ou[1], ou[2], ou[3]);
  }
}

static int ew_grid(long long items) {
  long long b = (items + 255) / 256;
  if (b > 148 * 16) b = 148 * 16;
  if (b < 1) b = 1;
  return (int)b;
}

}  // namespace nkb

using namespace nkb;

extern "C" int nkb_rope(void* qkv, int T, int S, int H, int D, float base, int backward,
                        int pos_offset, void* stream) {
  if (D % 16) return -3;
  long long items = (long long)T * 2 * H * (D / 16);
  rope_kernel<<<ew_grid(items), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<__nv_bfloat16*>(qkv), T, S, H, D, base, backward ? -1.f : 1.f, pos_offset);
  return (int)cudaGetLastError();
}

extern "C" int nkb_swiglu_fwd(const void* gu, void* h, long long T, int F, void* stream) {
  if (F % 8) return -3;
  swiglu_fwd_kernel<<<ew_grid(T * (F / 8)), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(gu), static_cast<__nv_bfloat16*>(h), T, F);
  return (int)cudaGetLastError();
}

extern "C" int nkb_swiglu_bwd(const void* gu, const void* dh, void* dgu, long long T, int F,
                              void* stream) {
  if (F % 8) return -3;
  swiglu_bwd_kernel<<<ew_grid(T * (F / 8)), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(gu), static_cast<const __nv_bfloat16*>(dh),
      static_cast<__nv_bfloat16*>(dgu), T, F);
  return (int)cudaGetLastError();
}
