// What joins the branches of a layer whose sublayers read one norm's output and are added at once, times a constant:
//   llmi_normed_pair       y[t] (+)= c * (a[t] / rms(a[t]) * wa + b[t] / rms(b[t]) * wb) — two mixers side by side, each
//                          normed over the model width with a weight of its own, then averaged (c = 1/2)
//   llmi_stream_axpy_norm  x[t] += m * y[t], and (optionally) h[t] = norm_w * x[t] / rms(x[t]) of the new x in the same
//                          pass: the norm ahead of the next layer
// rms(v) = sqrt(mean(v^2) + eps).  All arithmetic fp32; a block per row, rows are treated alone.
#include <math.h>

#include "common.cuh"

namespace llmi {

__device__ __forceinline__ void store4(float* o, float a, float b, float c, float d) {
  *reinterpret_cast<float4*>(o) = make_float4(a, b, c, d);
}
__device__ __forceinline__ void store4(__nv_bfloat16* o, float a, float b, float c, float d) {
  const __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
  uint2 u;
  u.x = *reinterpret_cast<const uint32_t*>(&lo);
  u.y = *reinterpret_cast<const uint32_t*>(&hi);
  *reinterpret_cast<uint2*>(o) = u;
}

__global__ void __launch_bounds__(256)
normed_pair_kernel(const float* __restrict__ a, long lda, const float* __restrict__ wa, const float* __restrict__ b, long ldb,
                   const float* __restrict__ wb, float eps, float coeff, float* __restrict__ y, long ldy, int W, int add,
                   int vec4) {
  __shared__ float scratch[32];
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const float* ar = a + (size_t)t * lda;
  const float* br = b + (size_t)t * ldb;
  float* yr = y + (size_t)t * ldy;
  float sa = 0.f, sb = 0.f;
  if (vec4) {                // rows of whole 16-byte pieces, every row starting on one
    for (int i = threadIdx.x; i < W / 4; i += blockDim.x) {
      const float4 p = reinterpret_cast<const float4*>(ar)[i], q = reinterpret_cast<const float4*>(br)[i];
      sa = fmaf(p.x, p.x, sa); sa = fmaf(p.y, p.y, sa); sa = fmaf(p.z, p.z, sa); sa = fmaf(p.w, p.w, sa);
      sb = fmaf(q.x, q.x, sb); sb = fmaf(q.y, q.y, sb); sb = fmaf(q.z, q.z, sb); sb = fmaf(q.w, q.w, sb);
    }
  } else {
    for (int i = threadIdx.x; i < W; i += blockDim.x) {
      sa = fmaf(ar[i], ar[i], sa);
      sb = fmaf(br[i], br[i], sb);
    }
  }
  sa = block_sum(sa, scratch);
  __syncthreads();
  sb = block_sum(sb, scratch);
  const float ia = 1.0f / sqrtf(sa / (float)W + eps), ib = 1.0f / sqrtf(sb / (float)W + eps);
  if (vec4) {
    for (int i = threadIdx.x; i < W / 4; i += blockDim.x) {
      const float4 p = reinterpret_cast<const float4*>(ar)[i], q = reinterpret_cast<const float4*>(br)[i];
      const float4 u = reinterpret_cast<const float4*>(wa)[i], w = reinterpret_cast<const float4*>(wb)[i];
      float4 v = make_float4(coeff * (p.x * ia * u.x + q.x * ib * w.x), coeff * (p.y * ia * u.y + q.y * ib * w.y),
                             coeff * (p.z * ia * u.z + q.z * ib * w.z), coeff * (p.w * ia * u.w + q.w * ib * w.w));
      if (add) {
        const float4 o = reinterpret_cast<const float4*>(yr)[i];
        v.x += o.x; v.y += o.y; v.z += o.z; v.w += o.w;
      }
      reinterpret_cast<float4*>(yr)[i] = v;
    }
  } else {
    for (int i = threadIdx.x; i < W; i += blockDim.x) {
      const float v = coeff * (ar[i] * ia * wa[i] + br[i] * ib * wb[i]);
      yr[i] = add ? yr[i] + v : v;
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(256)
stream_axpy_norm_kernel(float* __restrict__ x, const float* __restrict__ y, float m, int W, const float* __restrict__ norm_w,
                        float eps, T* __restrict__ h) {
  __shared__ float scratch[32];
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  float* xr = x + (size_t)t * W;
  const float* yr = y + (size_t)t * W;
  float ss = 0.f;
  if (W % 4 == 0) {          // rows of whole 16-byte pieces (x, y are contiguous: every row starts on one)
    for (int i = threadIdx.x; i < W / 4; i += blockDim.x) {
      float4 v = reinterpret_cast<const float4*>(xr)[i];
      const float4 u = reinterpret_cast<const float4*>(yr)[i];
      v.x = fmaf(m, u.x, v.x); v.y = fmaf(m, u.y, v.y); v.z = fmaf(m, u.z, v.z); v.w = fmaf(m, u.w, v.w);
      reinterpret_cast<float4*>(xr)[i] = v;
      ss = fmaf(v.x, v.x, ss); ss = fmaf(v.y, v.y, ss); ss = fmaf(v.z, v.z, ss); ss = fmaf(v.w, v.w, ss);
    }
  } else {
    for (int i = threadIdx.x; i < W; i += blockDim.x) {
      const float v = fmaf(m, yr[i], xr[i]);
      xr[i] = v;
      ss = fmaf(v, v, ss);
    }
  }
  if (!norm_w) return;
  ss = block_sum(ss, scratch);
  const float scale = 1.0f / sqrtf(ss / (float)W + eps);
  T* hr = h + (size_t)t * W;
  if (W % 4 == 0) {
    for (int i = threadIdx.x; i < W / 4; i += blockDim.x) {          // (my own writes above)
      const float4 v = reinterpret_cast<const float4*>(xr)[i], w = reinterpret_cast<const float4*>(norm_w)[i];
      store4(hr + 4 * i, w.x * (v.x * scale), w.y * (v.y * scale), w.z * (v.z * scale), w.w * (v.w * scale));
    }
  } else {
    for (int i = threadIdx.x; i < W; i += blockDim.x) hr[i] = from_f32<T>(norm_w[i] * (xr[i] * scale));
  }
}

}  // namespace llmi

using namespace llmi;

// a, b fp32 rows [T, lda / ldb] of W entries; wa, wb fp32 [W]; y fp32 [T, ldy] receives (add == 0) or gains the result.
LLMI_EXPORT int llmi_normed_pair(const float* a, long lda, const float* wa, const float* b, long ldb, const float* wb, float eps,
                                 float coeff, float* y, long ldy, int W, int n_rows, int add, cudaStream_t stream) {
  if (n_rows <= 0 || W <= 0) return LLMI_ERR_BAD_SIZE;
  const int threads = W >= 1024 ? 256 : (W >= 256 ? 128 : 64);
  const int vec4 = W % 4 == 0 && lda % 4 == 0 && ldb % 4 == 0 && ldy % 4 == 0 && !((uintptr_t)a & 15) && !((uintptr_t)b & 15) &&
                   !((uintptr_t)y & 15) && !((uintptr_t)wa & 15) && !((uintptr_t)wb & 15);
  return launch_pdl(PDL_SMALL, normed_pair_kernel, dim3(n_rows), dim3(threads), 0, stream, a, lda, wa, b, ldb, wb, eps, coeff, y, ldy,
                    W, add, vec4);
}

// x, y fp32 [T, W] contiguous: x += m * y.  With norm_w (fp32 [W]): h [T, W] contiguous in `dtype` = the RMS norm of the
// new x with that weight (computed as the norm kernel does: weight * (x * scale), rounded once).
LLMI_EXPORT int llmi_stream_axpy_norm(float* x, const float* y, float m, int n_rows, int W, const float* norm_w, float eps,
                                      int dtype, void* h, cudaStream_t stream) {
  if (n_rows <= 0 || W <= 0 || (norm_w && !h)) return LLMI_ERR_BAD_SIZE;
  if (W % 4 == 0 && (((uintptr_t)x & 15) || ((uintptr_t)y & 15) || ((uintptr_t)norm_w & 15) || ((uintptr_t)h & 15))) return LLMI_ERR_ALIGN;
  const int threads = W >= 1024 ? 256 : (W >= 256 ? 128 : 64);
  if (!norm_w || dtype == LLMI_DTYPE_F32)
    return launch_pdl(PDL_SMALL, stream_axpy_norm_kernel<float>, dim3(n_rows), dim3(threads), 0, stream, x, y, m, W, norm_w, eps,
                      (float*)h);
  if (dtype == LLMI_DTYPE_BF16)
    return launch_pdl(PDL_SMALL, stream_axpy_norm_kernel<__nv_bfloat16>, dim3(n_rows), dim3(threads), 0, stream, x, y, m, W, norm_w,
                      eps, (__nv_bfloat16*)h);
  return LLMI_ERR_BAD_DTYPE;
}
