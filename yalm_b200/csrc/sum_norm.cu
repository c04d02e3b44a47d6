// Row-wise kernels of layers that norm AFTER the residual sum:
//  * sum_norm: x <- n(alpha x + sum_b scale_b u_b, w), where each u_b is the sum of the split-K
//    slices of one product and may itself be normed over the row with a weight of its own
//    (two sublayers side by side whose outputs are normed before they are added);
//    n(v, w) = v / sqrt(mean(v^2) + eps) * w.  The new x is written back in 32 bits and, beside
//    it, in the compute type (the next sublayer's input);
//  * cast_rows: 32-bit rows in the compute type (the first layer's input);
//  * head_norm: every head's slice of a row normed over the head's size with one shared weight.
// All arithmetic is 32-bit.
#include "api.h"
#include "common.cuh"

namespace yalm {

struct SumBranch {
  const float* p;          // [n][rows][dim] slices
  int n;
  long long stride;
  const float* w;          // null: the branch is added as it is
  float scale;
};

constexpr int SN_VPT = 8;    // elements of a row a thread keeps (rows of up to 8 x 1024)

template <typename TO>
__global__ void __launch_bounds__(1024)
sum_norm_kernel(float* __restrict__ x, float alpha, SumBranch b0, SumBranch b1, int n_branches,
                float branch_eps, const float* __restrict__ weight, float eps, TO* __restrict__ h,
                int dim) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float scratch[33];
  const int r = blockIdx.x;
  float* xr = x + (size_t)r * dim;
  float u0[SN_VPT], u1[SN_VPT], v[SN_VPT];
  float ss0 = 0.f, ss1 = 0.f;
#pragma unroll
  for (int k = 0; k < SN_VPT; ++k) {
    const int i = threadIdx.x + k * blockDim.x;
    u0[k] = u1[k] = 0.f;
    if (i < dim) {
      if (n_branches > 0) u0[k] = sum_slices(b0.p + (size_t)r * dim + i, b0.n, b0.stride);
      if (n_branches > 1) u1[k] = sum_slices(b1.p + (size_t)r * dim + i, b1.n, b1.stride);
    }
    ss0 += u0[k] * u0[k];
    ss1 += u1[k] * u1[k];
  }
  float rs0 = 1.f, rs1 = 1.f;
  if (n_branches > 0 && b0.w != nullptr) rs0 = 1.0f / sqrtf(block_sum(ss0, scratch) / (float)dim + branch_eps);
  if (n_branches > 1 && b1.w != nullptr) rs1 = 1.0f / sqrtf(block_sum(ss1, scratch) / (float)dim + branch_eps);
  float ss = 0.f;
#pragma unroll
  for (int k = 0; k < SN_VPT; ++k) {
    const int i = threadIdx.x + k * blockDim.x;
    v[k] = 0.f;
    if (i < dim) {
      float a = n_branches > 0 ? (b0.w != nullptr ? u0[k] * rs0 * b0.w[i] : u0[k]) * b0.scale : 0.f;
      if (n_branches > 1) a += (b1.w != nullptr ? u1[k] * rs1 * b1.w[i] : u1[k]) * b1.scale;
      v[k] = fmaf(alpha, xr[i], a);
    }
    ss += v[k] * v[k];
  }
  const float rs = 1.0f / sqrtf(block_sum(ss, scratch) / (float)dim + eps);
#pragma unroll
  for (int k = 0; k < SN_VPT; ++k) {
    const int i = threadIdx.x + k * blockDim.x;
    if (i < dim) {
      const float y = v[k] * rs * weight[i];
      xr[i] = y;
      if (h != nullptr) h[(size_t)r * dim + i] = from_float<TO>(y);
    }
  }
}

// The same with four neighbouring features per thread and step (dim % 4 == 0, 16-byte aligned
// pointers): every load of a pass is in flight at once.
__device__ __forceinline__ float4 ld4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 sum_slices4(const float* p, int n, long long stride) {
  float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int s0 = 0; s0 < n; s0 += 4) {
    float4 t[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) t[j] = s0 + j < n ? ld4(p + (size_t)(s0 + j) * stride) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int j = 0; j < 4; ++j) { v.x += t[j].x; v.y += t[j].y; v.z += t[j].z; v.w += t[j].w; }
  }
  return v;
}
__device__ __forceinline__ float sq4(float4 v) { return v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w; }
__device__ __forceinline__ void st4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
template <typename T16> __device__ __forceinline__ void st4(T16* p, float4 v) {
  uint2 u;
  u.x = pack2<T16>(v.x, v.y);
  u.y = pack2<T16>(v.z, v.w);
  *reinterpret_cast<uint2*>(p) = u;
}

template <typename TO, int VPT>
__global__ void __launch_bounds__(1024)
sum_norm_vec_kernel(float* __restrict__ x, float alpha, SumBranch b0, SumBranch b1, int n_branches,
                    float branch_eps, const float* __restrict__ weight, float eps, TO* __restrict__ h,
                    int dim) {
  pdl_launch_dependents();
  const int nvec = dim >> 2;
  float4 w[VPT];
#pragma unroll
  for (int k = 0; k < VPT; ++k) {                       // the weights do not depend on the previous kernel
    const int c = threadIdx.x + k * blockDim.x;
    w[k] = c < nvec ? ld4(weight + 4 * c) : make_float4(0.f, 0.f, 0.f, 0.f);
  }
  pdl_wait();
  __shared__ float scratch[33];
  const size_t r0 = (size_t)blockIdx.x * dim;
  const float4 zero = make_float4(0.f, 0.f, 0.f, 0.f);
  float4 u0[VPT], u1[VPT], v[VPT];
  float ss0 = 0.f, ss1 = 0.f;
#pragma unroll
  for (int k = 0; k < VPT; ++k) {
    const int c = threadIdx.x + k * blockDim.x;
    u0[k] = (n_branches > 0 && c < nvec) ? sum_slices4(b0.p + r0 + 4 * c, b0.n, b0.stride) : zero;
    u1[k] = (n_branches > 1 && c < nvec) ? sum_slices4(b1.p + r0 + 4 * c, b1.n, b1.stride) : zero;
    v[k] = c < nvec ? ld4(x + r0 + 4 * c) : zero;
    ss0 += sq4(u0[k]);
    ss1 += sq4(u1[k]);
  }
  float rs0 = 1.f, rs1 = 1.f;
  if (n_branches > 0 && b0.w != nullptr) rs0 = 1.0f / sqrtf(block_sum(ss0, scratch) / (float)dim + branch_eps);
  if (n_branches > 1 && b1.w != nullptr) rs1 = 1.0f / sqrtf(block_sum(ss1, scratch) / (float)dim + branch_eps);
  float ss = 0.f;
#pragma unroll
  for (int k = 0; k < VPT; ++k) {
    const int c = threadIdx.x + k * blockDim.x;
    if (c < nvec) {
      float4 a = zero;
      if (n_branches > 0) {
        float4 t = u0[k];
        if (b0.w != nullptr) {
          const float4 bw = ld4(b0.w + 4 * c);
          t = make_float4(t.x * rs0 * bw.x, t.y * rs0 * bw.y, t.z * rs0 * bw.z, t.w * rs0 * bw.w);
        }
        a = make_float4(t.x * b0.scale, t.y * b0.scale, t.z * b0.scale, t.w * b0.scale);
      }
      if (n_branches > 1) {
        float4 t = u1[k];
        if (b1.w != nullptr) {
          const float4 bw = ld4(b1.w + 4 * c);
          t = make_float4(t.x * rs1 * bw.x, t.y * rs1 * bw.y, t.z * rs1 * bw.z, t.w * rs1 * bw.w);
        }
        a.x += t.x * b1.scale; a.y += t.y * b1.scale; a.z += t.z * b1.scale; a.w += t.w * b1.scale;
      }
      v[k] = make_float4(fmaf(alpha, v[k].x, a.x), fmaf(alpha, v[k].y, a.y), fmaf(alpha, v[k].z, a.z),
                         fmaf(alpha, v[k].w, a.w));
    }
    ss += sq4(v[k]);
  }
  const float rs = 1.0f / sqrtf(block_sum(ss, scratch) / (float)dim + eps);
#pragma unroll
  for (int k = 0; k < VPT; ++k) {
    const int c = threadIdx.x + k * blockDim.x;
    if (c < nvec) {
      const float4 y = make_float4(v[k].x * rs * w[k].x, v[k].y * rs * w[k].y, v[k].z * rs * w[k].z,
                                   v[k].w * rs * w[k].w);
      st4(x + r0 + 4 * c, y);
      if (h != nullptr) st4(h + r0 + 4 * c, y);
    }
  }
}

template <typename TO>
__global__ void cast_rows_kernel(const float* __restrict__ x, TO* __restrict__ out, long long n) {
  pdl_launch_dependents();
  pdl_wait();
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x)
    out[i] = from_float<TO>(x[i]);
}

// One warp per (row, head): out[row, head, :] = n(o[row, head, :], w) over the head's `size` values.
template <typename TO>
__global__ void head_norm_kernel(const float* __restrict__ o, const float* __restrict__ w,
                                 TO* __restrict__ out, long long n_heads_total, int size, float eps) {
  pdl_launch_dependents();
  pdl_wait();
  const long long head = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (head >= n_heads_total) return;
  const int lane = threadIdx.x & 31;
  const float* src = o + head * size;
  float ss = 0.f;
  for (int i = lane; i < size; i += 32) ss += src[i] * src[i];
  ss = warp_sum(ss);
  const float rs = 1.0f / sqrtf(ss / (float)size + eps);
  for (int i = lane; i < size; i += 32) out[head * size + i] = from_float<TO>(src[i] * rs * w[i]);
}

}  // namespace yalm

using namespace yalm;

// x [rows, dim] <- n(alpha x + scale0 B0 + scale1 B1, weight); Bj is the sum of nj slices
// (stride between slices: sj floats), normed over the row with wj (and branch_eps) when wj is
// not null.  h (null, or [rows, dim] of h_dtype) receives the new x in that type.
extern "C" int yalm_sum_norm(float* x, float alpha, int n_branches, const float* p0, int n0,
                             long long s0, const float* w0, float scale0, const float* p1, int n1,
                             long long s1, const float* w1, float scale1, float branch_eps,
                             const float* weight, float eps, void* h, int h_dtype, int rows, int dim,
                             cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (dim <= 0 || dim > SN_VPT * 1024 || n_branches < 0 || n_branches > 2) return -2;
  SumBranch b0 = {p0, n0, s0, w0, scale0}, b1 = {p1, n1, s1, w1, scale1};
  int threads = (dim + SN_VPT - 1) / SN_VPT;
  threads = (threads + 31) / 32 * 32;
  if (threads < 128 && dim >= 128) threads = 128;
  if (rows <= 256) {                                  // a few rows: one element per thread where that fits
    threads = (dim + 31) / 32 * 32;
    if (threads > 1024) threads = 1024;
  }
  const bool vec = dim % 4 == 0 && s0 % 4 == 0 && s1 % 4 == 0 &&
                   ((((uintptr_t)x) | ((uintptr_t)p0) | ((uintptr_t)p1) | ((uintptr_t)w0) | ((uintptr_t)w1) |
                     ((uintptr_t)weight) | ((uintptr_t)h)) & 15) == 0;
  if (vec) {
    const int nvec = dim / 4;
    int vt;                                             // few rows: one vector per thread; many: two
    if (rows <= 256 || nvec <= 256) vt = nvec <= 1024 ? (nvec + 31) / 32 * 32 : 1024;
    else vt = ((nvec + 1) / 2 + 31) / 32 * 32;
    if (vt > 1024) vt = 1024;
    const int vpt = (nvec + vt - 1) / vt;
    void* hh = (h == nullptr) ? nullptr : h;
#define YALM_SNV(T, V)                                                                                 \
  launch_pdl(sum_norm_vec_kernel<T, V>, dim3(rows), dim3(vt), 0, stream, x, alpha, b0, b1, n_branches, \
             branch_eps, weight, eps, (T*)hh, dim)
    const int dt = h == nullptr ? DT_F32 : h_dtype;
    if (dt == DT_F32) { if (vpt <= 1) YALM_SNV(float, 1); else YALM_SNV(float, 2); }
    else if (dt == DT_BF16) { if (vpt <= 1) YALM_SNV(__nv_bfloat16, 1); else YALM_SNV(__nv_bfloat16, 2); }
    else if (dt == DT_F16) { if (vpt <= 1) YALM_SNV(__half, 1); else YALM_SNV(__half, 2); }
    else return -3;
#undef YALM_SNV
    YALM_LAUNCH_CHECK();
    return 0;
  }
  const dim3 grid(rows), block(threads);
  if (h == nullptr || h_dtype == DT_F32)
    launch_pdl(sum_norm_kernel<float>, grid, block, 0, stream, x, alpha, b0, b1, n_branches, branch_eps,
               weight, eps, (float*)(h_dtype == DT_F32 ? h : nullptr), dim);
  else if (h_dtype == DT_BF16)
    launch_pdl(sum_norm_kernel<__nv_bfloat16>, grid, block, 0, stream, x, alpha, b0, b1, n_branches,
               branch_eps, weight, eps, (__nv_bfloat16*)h, dim);
  else if (h_dtype == DT_F16)
    launch_pdl(sum_norm_kernel<__half>, grid, block, 0, stream, x, alpha, b0, b1, n_branches, branch_eps,
               weight, eps, (__half*)h, dim);
  else
    return -3;
  YALM_LAUNCH_CHECK();
  return 0;
}

extern "C" int yalm_cast_rows(const float* x, void* out, int out_dtype, long long n, cudaStream_t stream) {
  if (n <= 0) return 0;
  long long blocks = (n + 255) / 256;
  if (blocks > 148 * 32) blocks = 148 * 32;
  const dim3 grid((unsigned)blocks), block(256);
  if (out_dtype == DT_BF16) launch_pdl(cast_rows_kernel<__nv_bfloat16>, grid, block, 0, stream, x, (__nv_bfloat16*)out, n);
  else if (out_dtype == DT_F16) launch_pdl(cast_rows_kernel<__half>, grid, block, 0, stream, x, (__half*)out, n);
  else if (out_dtype == DT_F32) launch_pdl(cast_rows_kernel<float>, grid, block, 0, stream, x, (float*)out, n);
  else return -3;
  YALM_LAUNCH_CHECK();
  return 0;
}

// out [rows, heads * size] (out_dtype) = every head's `size` values of o (float32) normed with w [size]
extern "C" int yalm_head_norm(const float* o, const float* w, void* out, int out_dtype, long long rows,
                              int heads, int size, float eps, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (heads <= 0 || size <= 0) return -2;
  const long long total = rows * heads;
  const long long blocks = (total + 7) / 8;
  if (blocks > 0x7fffffffLL) return -4;
  const dim3 grid((unsigned)blocks), block(256);
  if (out_dtype == DT_BF16)
    launch_pdl(head_norm_kernel<__nv_bfloat16>, grid, block, 0, stream, o, w, (__nv_bfloat16*)out, total, size, eps);
  else if (out_dtype == DT_F16)
    launch_pdl(head_norm_kernel<__half>, grid, block, 0, stream, o, w, (__half*)out, total, size, eps);
  else if (out_dtype == DT_F32)
    launch_pdl(head_norm_kernel<float>, grid, block, 0, stream, o, w, (float*)out, total, size, eps);
  else
    return -3;
  YALM_LAUNCH_CHECK();
  return 0;
}
