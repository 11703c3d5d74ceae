// Row-wise pieces that act on the fp32 residual stream of a step.
//
//   llmi_layernorm    y = (x - mean) / sqrt(var + eps) * w  (a weight, no bias; var = mean of the squared deviations),
//                     for one weight or for TWO weights at once: a layer that reads the same x through two norms shares
//                     the row's mean and variance, so both outputs leave from one read of x.  `rows` (optional) picks
//                     the input row of each output row (-1: zeros).
//   llmi_depth_mix    files the stream as a layer leaves it in a record of the step, hist[n] = x, and replaces the
//                     stream by a learned mixture over the depth so far:  x = sum_{j <= n} c[j] * hist[j]  (j ascending).
//   llmi_gate_rows    a[t, :] *= sigmoid(z[t]) — one number per token on a whole row (in the row's type).
//   llmi_mix_layernorm  both of the above for a row in one pass (a block per row, the row in registers): the record and
//                     the mixture as llmi_depth_mix makes them (same order of additions), then one or two layer norms of
//                     the mixed row.  With n < 0 nothing is mixed: the layer norm alone, for widths a warp is too few for.
// All sums in fp32; rows are treated alone.
#include <math.h>

#include "common.cuh"

namespace llmi {

__device__ __forceinline__ void ln_store4(float* o, float a, float b, float c, float d) {
  *reinterpret_cast<float4*>(o) = make_float4(a, b, c, d);
}
__device__ __forceinline__ void ln_store4(__nv_bfloat16* o, float a, float b, float c, float d) {
  const __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
  uint2 u;
  u.x = *reinterpret_cast<const uint32_t*>(&lo);
  u.y = *reinterpret_cast<const uint32_t*>(&hi);
  *reinterpret_cast<uint2*>(o) = u;
}

// One warp per row, the row in registers (VPT 16-byte loads a lane): mean, then the squared deviations, then the outputs.
template <typename T, int VPT>
__global__ void __launch_bounds__(256)
layernorm_warp_kernel(const float* __restrict__ x, const float* __restrict__ w1, T* __restrict__ out1,
                      const float* __restrict__ w2, T* __restrict__ out2, const int32_t* __restrict__ rows, int n_rows,
                      int width, float eps) {
  pdl_launch_dependents();
  pdl_wait();
  const int r = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (r >= n_rows) return;
  const int src = rows ? rows[r] : r;
  const int nvec = width >> 2;
  float4 v[VPT];
  float s = 0.f;
#pragma unroll
  for (int j = 0; j < VPT; ++j) {
    const int i = lane + j * 32;
    v[j] = (src >= 0 && i < nvec) ? reinterpret_cast<const float4*>(x + (size_t)src * width)[i] : make_float4(0.f, 0.f, 0.f, 0.f);
    s += (v[j].x + v[j].y) + (v[j].z + v[j].w);
  }
  const float mean = warp_sum(s) / (float)width;
  float q = 0.f;
#pragma unroll
  for (int j = 0; j < VPT; ++j) {
    const int i = lane + j * 32;
    if (i < nvec) {
      v[j].x -= mean; v[j].y -= mean; v[j].z -= mean; v[j].w -= mean;
      q = fmaf(v[j].x, v[j].x, fmaf(v[j].y, v[j].y, fmaf(v[j].z, v[j].z, fmaf(v[j].w, v[j].w, q))));
    }
  }
  const float rstd = src >= 0 ? 1.0f / sqrtf(warp_sum(q) / (float)width + eps) : 0.f;
#pragma unroll
  for (int j = 0; j < VPT; ++j) {
    const int i = lane + j * 32;
    if (i < nvec) {
      const float4 a = reinterpret_cast<const float4*>(w1)[i];
      ln_store4(out1 + (size_t)r * width + 4 * i, v[j].x * rstd * a.x, v[j].y * rstd * a.y, v[j].z * rstd * a.z, v[j].w * rstd * a.w);
      if (w2) {
        const float4 b = reinterpret_cast<const float4*>(w2)[i];
        ln_store4(out2 + (size_t)r * width + 4 * i, v[j].x * rstd * b.x, v[j].y * rstd * b.y, v[j].z * rstd * b.z, v[j].w * rstd * b.w);
      }
    }
  }
}

// Any width: one block per row, x read three times (the row stays in the caches).
template <typename T>
__global__ void __launch_bounds__(256)
layernorm_block_kernel(const float* __restrict__ x, const float* __restrict__ w1, T* __restrict__ out1,
                       const float* __restrict__ w2, T* __restrict__ out2, const int32_t* __restrict__ rows, int width, float eps) {
  __shared__ float scratch[32];
  pdl_launch_dependents();
  pdl_wait();
  const int r = blockIdx.x;
  const int src = rows ? rows[r] : r;
  T* o1 = out1 + (size_t)r * width;
  T* o2 = w2 ? out2 + (size_t)r * width : nullptr;
  if (src < 0) {
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
      o1[i] = from_f32<T>(0.f);
      if (o2) o2[i] = from_f32<T>(0.f);
    }
    return;
  }
  const float* xr = x + (size_t)src * width;
  float s = 0.f;
  for (int i = threadIdx.x; i < width; i += blockDim.x) s += xr[i];
  const float mean = block_sum(s, scratch) / (float)width;
  float q = 0.f;
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    const float d = xr[i] - mean;
    q = fmaf(d, d, q);
  }
  const float rstd = 1.0f / sqrtf(block_sum(q, scratch) / (float)width + eps);
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    const float d = (xr[i] - mean) * rstd;
    o1[i] = from_f32<T>(d * w1[i]);
    if (o2) o2[i] = from_f32<T>(d * w2[i]);
  }
}

// One block per row, VPT 16-byte pieces a thread.  n >= 0: hist[n] = x; x = sum_{j<=n} c[j] hist[j] (j ascending, one fma
// chain from 0, as depth_mix_kernel adds them), then the norms of the new x.  n < 0: the norms of x (rows: which row each
// output row reads, -1: zeros; only without a mixture).
template <typename T, int VPT, int THREADS>
__global__ void __launch_bounds__(THREADS)
mix_layernorm_kernel(float* __restrict__ x, float* __restrict__ hist, long row_floats, int n, const float* __restrict__ c,
                     const float* __restrict__ w1, T* __restrict__ out1, const float* __restrict__ w2, T* __restrict__ out2,
                     const int32_t* __restrict__ rows, int width, float eps) {
  __shared__ float scratch[32];
  pdl_launch_dependents();
  pdl_wait();
  const int r = blockIdx.x;
  const int src = (rows && n < 0) ? rows[r] : r;
  const int nvec = width >> 2;
  float4 v[VPT], wa[VPT], wb[VPT];
  // the weights first: nothing below waits for them until the row's sums are done
#pragma unroll
  for (int j = 0; j < VPT; ++j) {
    const int i = threadIdx.x + j * THREADS;
    wa[j] = wb[j] = make_float4(0.f, 0.f, 0.f, 0.f);
    if (i < nvec) {
      wa[j] = reinterpret_cast<const float4*>(w1)[i];
      if (w2) wb[j] = reinterpret_cast<const float4*>(w2)[i];
    }
  }
  float s = 0.f;
#pragma unroll
  for (int j = 0; j < VPT; ++j) {
    const int i = threadIdx.x + j * THREADS;
    v[j] = make_float4(0.f, 0.f, 0.f, 0.f);
    if (src >= 0 && i < nvec) {
      const size_t at = (size_t)src * nvec + i;
      const float4 cur = reinterpret_cast<const float4*>(x)[at];
      if (n >= 0) {
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        int k = 0;
        for (; k + 4 <= n; k += 4) {          // four rows of the record in flight at a time; added in the order of k
          float4 h[4];
#pragma unroll
          for (int u = 0; u < 4; ++u) h[u] = __ldcg(reinterpret_cast<const float4*>(hist + (size_t)(k + u) * row_floats) + at);
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            const float ck = c[k + u];
            acc.x = fmaf(ck, h[u].x, acc.x); acc.y = fmaf(ck, h[u].y, acc.y); acc.z = fmaf(ck, h[u].z, acc.z); acc.w = fmaf(ck, h[u].w, acc.w);
          }
        }
        for (; k < n; ++k) {
          const float4 h = __ldcg(reinterpret_cast<const float4*>(hist + (size_t)k * row_floats) + at);
          const float ck = c[k];
          acc.x = fmaf(ck, h.x, acc.x); acc.y = fmaf(ck, h.y, acc.y); acc.z = fmaf(ck, h.z, acc.z); acc.w = fmaf(ck, h.w, acc.w);
        }
        const float cn = c[n];
        acc.x = fmaf(cn, cur.x, acc.x); acc.y = fmaf(cn, cur.y, acc.y); acc.z = fmaf(cn, cur.z, acc.z); acc.w = fmaf(cn, cur.w, acc.w);
        reinterpret_cast<float4*>(hist + (size_t)n * row_floats)[at] = cur;
        reinterpret_cast<float4*>(x)[at] = acc;
        v[j] = acc;
      } else {
        v[j] = cur;
      }
    }
    s += (v[j].x + v[j].y) + (v[j].z + v[j].w);
  }
  const float mean = block_sum(s, scratch) / (float)width;
  float q = 0.f;
#pragma unroll
  for (int j = 0; j < VPT; ++j) {
    const int i = threadIdx.x + j * THREADS;
    if (i < nvec) {
      v[j].x -= mean; v[j].y -= mean; v[j].z -= mean; v[j].w -= mean;
      q = fmaf(v[j].x, v[j].x, fmaf(v[j].y, v[j].y, fmaf(v[j].z, v[j].z, fmaf(v[j].w, v[j].w, q))));
    }
  }
  const float rstd = src >= 0 ? 1.0f / sqrtf(block_sum(q, scratch) / (float)width + eps) : 0.f;
#pragma unroll
  for (int j = 0; j < VPT; ++j) {
    const int i = threadIdx.x + j * THREADS;
    if (i < nvec) {
      const float4 a = wa[j];
      ln_store4(out1 + (size_t)r * width + 4 * i, v[j].x * rstd * a.x, v[j].y * rstd * a.y, v[j].z * rstd * a.z, v[j].w * rstd * a.w);
      if (w2) {
        const float4 b = wb[j];
        ln_store4(out2 + (size_t)r * width + 4 * i, v[j].x * rstd * b.x, v[j].y * rstd * b.y, v[j].z * rstd * b.z, v[j].w * rstd * b.w);
      }
    }
  }
}

// n: rows of the record that are there before this call (hist[0 .. n-1]); the stream becomes row n.
__global__ void __launch_bounds__(256)
depth_mix_kernel(float* __restrict__ x, float* __restrict__ hist, long row_floats, int n, const float* __restrict__ c, long n4,
                 long total) {
  pdl_launch_dependents();
  pdl_wait();
  const long i = (long)blockIdx.x * blockDim.x + threadIdx.x;
  if (n4 > 0) {
    if (i >= n4) return;
    const float4 cur = reinterpret_cast<const float4*>(x)[i];
    reinterpret_cast<float4*>(hist + (size_t)n * row_floats)[i] = cur;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int j = 0; j < n; ++j) {
      const float4 h = reinterpret_cast<const float4*>(hist + (size_t)j * row_floats)[i];
      const float cj = c[j];
      acc.x = fmaf(cj, h.x, acc.x); acc.y = fmaf(cj, h.y, acc.y); acc.z = fmaf(cj, h.z, acc.z); acc.w = fmaf(cj, h.w, acc.w);
    }
    const float cn = c[n];
    acc.x = fmaf(cn, cur.x, acc.x); acc.y = fmaf(cn, cur.y, acc.y); acc.z = fmaf(cn, cur.z, acc.z); acc.w = fmaf(cn, cur.w, acc.w);
    reinterpret_cast<float4*>(x)[i] = acc;
  } else {
    if (i >= total) return;
    const float cur = x[i];
    hist[(size_t)n * row_floats + i] = cur;
    float acc = 0.f;
    for (int j = 0; j < n; ++j) acc = fmaf(c[j], hist[(size_t)j * row_floats + i], acc);
    x[i] = fmaf(c[n], cur, acc);
  }
}

template <typename T>
__global__ void __launch_bounds__(256)
gate_rows_kernel(T* __restrict__ a, long lda, int width, const float* __restrict__ z, long ldz, int n_rows) {
  pdl_launch_dependents();
  pdl_wait();
  const int r = blockIdx.x;
  const float g = 1.0f / (1.0f + expf(-z[(size_t)r * ldz]));
  T* row = a + (size_t)r * lda;
  for (int i = threadIdx.x; i < width; i += blockDim.x) row[i] = from_f32<T>(to_f32(row[i]) * g);
}

// widths of 4 .. 4096 floats in 16-byte pieces: 128 threads, up to 8 pieces each
template <typename T>
static int launch_mix_layernorm(float* x, float* hist, long row_floats, int n, const float* c, const float* w1, void* out1,
                                const float* w2, void* out2, const int32_t* rows, int n_rows, int width, float eps,
                                cudaStream_t stream) {
  const int vpt = (width / 4 + 127) / 128;
#define LLMI_MLN(V)                                                                                                          \
  return launch_pdl(PDL_SMALL, mix_layernorm_kernel<T, V, 128>, dim3(n_rows), dim3(128), 0, stream, x, hist, row_floats, n, c, w1, \
                    (T*)out1, w2, (T*)out2, rows, width, eps)
  if (vpt <= 1) LLMI_MLN(1);
  if (vpt <= 2) LLMI_MLN(2);
  if (vpt <= 4) LLMI_MLN(4);
  LLMI_MLN(8);
#undef LLMI_MLN
}

template <typename T>
static int launch_layernorm(const float* x, const float* w1, void* out1, const float* w2, void* out2, const int32_t* rows, int n_rows,
                            int width, float eps, cudaStream_t stream) {
  const bool aligned = (width % 4 == 0) && !((uintptr_t)x & 15) && !((uintptr_t)w1 & 15) && !((uintptr_t)out1 & 15) &&
                       !((uintptr_t)w2 & 15) && !((uintptr_t)out2 & 15);
  const int nvec = width / 4;
  if (aligned && nvec > 64 && nvec <= 128 * 8) return launch_mix_layernorm<T>(const_cast<float*>(x), nullptr, 0, -1, nullptr, w1, out1, w2, out2, rows, n_rows, width, eps, stream);
  if (aligned && nvec <= 32 * 16) {
    const int vpt = (nvec + 31) / 32;
    const unsigned blocks = (unsigned)((n_rows + 7) / 8);
#define LLMI_LN(V)                                                                                                        \
  return launch_pdl(PDL_SMALL, layernorm_warp_kernel<T, V>, dim3(blocks), dim3(256), 0, stream, x, w1, (T*)out1, w2, (T*)out2, rows, \
                    n_rows, width, eps)
    if (vpt <= 1) LLMI_LN(1);
    if (vpt <= 2) LLMI_LN(2);
    if (vpt <= 4) LLMI_LN(4);
    if (vpt <= 8) LLMI_LN(8);
    LLMI_LN(16);
#undef LLMI_LN
  }
  return launch_pdl(PDL_SMALL, layernorm_block_kernel<T>, dim3(n_rows), dim3(256), 0, stream, x, w1, (T*)out1, w2, (T*)out2, rows, width,
                    eps);
}

}  // namespace llmi

using namespace llmi;

// out2 / w2 may be null (one norm).  x fp32 [*, width]; outputs [n_rows, width] in out_dtype.
LLMI_EXPORT int llmi_layernorm(int out_dtype, const float* x, const float* w1, void* out1, const float* w2, void* out2,
                               const int32_t* rows, int n_rows, int width, float eps, cudaStream_t stream) {
  if (n_rows <= 0 || width <= 0 || !w1 || !out1 || ((w2 == nullptr) != (out2 == nullptr))) return LLMI_ERR_BAD_SIZE;
  if (out_dtype == LLMI_DTYPE_F32) return launch_layernorm<float>(x, w1, out1, w2, out2, rows, n_rows, width, eps, stream);
  if (out_dtype == LLMI_DTYPE_BF16) return launch_layernorm<__nv_bfloat16>(x, w1, out1, w2, out2, rows, n_rows, width, eps, stream);
  return LLMI_ERR_BAD_DTYPE;
}

// llmi_depth_mix followed by llmi_layernorm of every row of the new x, in one kernel.  x [n_rows, width] fp32 contiguous;
// hist entries `n_rows * width` floats apart.  LLMI_ERR_UNSUPPORTED where the fused form does not apply (the caller runs the two).
LLMI_EXPORT int llmi_mix_layernorm(int out_dtype, float* x, float* hist, int n, const float* c, const float* w1, void* out1,
                                   const float* w2, void* out2, int n_rows, int width, float eps, cudaStream_t stream) {
  if (n_rows <= 0 || width <= 0 || n < 0 || !w1 || !out1 || ((w2 == nullptr) != (out2 == nullptr))) return LLMI_ERR_BAD_SIZE;
  const bool aligned = (width % 4 == 0) && !((uintptr_t)x & 15) && !((uintptr_t)hist & 15) && !((uintptr_t)w1 & 15) &&
                       !((uintptr_t)out1 & 15) && !((uintptr_t)w2 & 15) && !((uintptr_t)out2 & 15);
  if (!aligned || width > 4096) return LLMI_ERR_UNSUPPORTED;
  const long row_floats = (long)n_rows * width;
  if (out_dtype == LLMI_DTYPE_F32)
    return launch_mix_layernorm<float>(x, hist, row_floats, n, c, w1, out1, w2, out2, nullptr, n_rows, width, eps, stream);
  if (out_dtype == LLMI_DTYPE_BF16)
    return launch_mix_layernorm<__nv_bfloat16>(x, hist, row_floats, n, c, w1, out1, w2, out2, nullptr, n_rows, width, eps, stream);
  return LLMI_ERR_BAD_DTYPE;
}

// x, hist rows: `row_floats` floats each (tokens * width); c: n + 1 coefficients on the device.
LLMI_EXPORT int llmi_depth_mix(float* x, float* hist, long row_floats, int n, const float* c, cudaStream_t stream) {
  if (row_floats <= 0 || n < 0) return LLMI_ERR_BAD_SIZE;
  const bool vec = (row_floats % 4 == 0) && !((uintptr_t)x & 15) && !((uintptr_t)hist & 15);
  const long n4 = vec ? row_floats / 4 : 0;
  const long work = vec ? n4 : row_floats;
  const long blocks = (work + 255) / 256;
  if (blocks > 0x7fffffffL) return LLMI_ERR_BAD_SIZE;
  return launch_pdl(PDL_SMALL, depth_mix_kernel, dim3((unsigned)blocks), dim3(256), 0, stream, x, hist, row_floats, n, c, n4, row_floats);
}

LLMI_EXPORT int llmi_gate_rows(int dtype, void* a, long lda, int width, const float* z, long ldz, int n_rows, cudaStream_t stream) {
  if (n_rows <= 0 || width <= 0) return LLMI_ERR_BAD_SIZE;
  if (dtype == LLMI_DTYPE_F32)
    return launch_pdl(PDL_SMALL, gate_rows_kernel<float>, dim3(n_rows), dim3(256), 0, stream, (float*)a, lda, width, z, ldz, n_rows);
  if (dtype == LLMI_DTYPE_BF16)
    return launch_pdl(PDL_SMALL, gate_rows_kernel<__nv_bfloat16>, dim3(n_rows), dim3(256), 0, stream, (__nv_bfloat16*)a, lda, width, z,
                      ldz, n_rows);
  return LLMI_ERR_BAD_DTYPE;
}
