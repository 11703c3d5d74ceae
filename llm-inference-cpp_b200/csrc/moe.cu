// Routed experts: each token runs `top` of E small gated feed-forwards, chosen by the largest router logits, and
// adds their outputs weighted by the softmax over the CHOSEN logits only.
//
//   llmi_moe_route    per token: the `top` largest of E fp32 logits (ties: the lower index), their softmax (fp32);
//                     or (`mode` 1) scores s = logistic(logit), the `top` largest scores weighted by s / (sum of the
//                     chosen s + 1e-20), optionally among the experts of the best `keep` of `n_groups` equal runs of
//                     neighbouring experts only, a run's score being the sum of its two largest scores;
//                     or (`mode` 2) scores s = softmax over ALL E logits, the choice by s + correction (a learned
//                     number per expert), the weights s * scale without a division by their sum.  In this mode the last
//                     `n_identity` of the E router outputs stand for experts that hand their input on: such a choice
//                     is written as index -1 (the product kernels skip it) and the token's summed weight of them to
//                     `id_wt`, for llmi_moe_identity_add
//   llmi_moe_up       per (token, choice): a = act(Wg_e h) * (Wu_e h), or a = act(Wu_e h) for experts
//                     without a gate matrix                                                  [T, top, F] fp32
//   llmi_moe_down     per token: y = sum over its choices, in the order of the choice, of weight * (Wd_e a)   [T, W] fp32
// The two product kernels stream an expert's rows once per (token, choice): the form for a handful of tokens (a
// decode step), where every chosen expert's weights are read once or a few times anyway.  Each output is one
// warp's sum in a fixed order, so a token's result does not depend on the batch it is in.
// Weights are stacked by expert: Wg, Wu [E, F, W], Wd [E, W, F], in the compute type; act: 0 silu, 1 tanh-GELU,
// 2 the square of relu.
#include <math.h>

#include "common.cuh"

namespace llmi {

constexpr int MOE_MAX_PER_LANE = 8;      // experts per lane: E <= 256

// The warp's best (value, index) pair; ties go to the lower index.  Every lane gets it.
__device__ __forceinline__ void warp_best(float& best, int& best_e) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ob = __shfl_xor_sync(0xffffffffu, best, o);
    const int oe = __shfl_xor_sync(0xffffffffu, best_e, o);
    if (ob > best || (ob == best && oe < best_e)) { best = ob; best_e = oe; }
  }
}

// One warp per token.  MODE 0: softmax over the chosen logits.  MODE 1: logistic scores, normalised over the chosen.
// MODE 2: softmax over all logits, chosen by score + correction, weighted by score * scale.
template <int MODE>
__global__ void __launch_bounds__(128)
moe_route_kernel(const float* __restrict__ logits, long ld, int E, int top, int n_groups, int keep,
                 const int32_t* __restrict__ tok_seq, int32_t* __restrict__ idx, float* __restrict__ wt, int n_tokens,
                 const float* __restrict__ correction, float scale, int n_identity, float* __restrict__ id_wt) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (t >= n_tokens) return;
  if (tok_seq[t] < 0) {
    for (int j = lane; j < top; j += 32) { idx[(size_t)t * top + j] = -1; wt[(size_t)t * top + j] = 0.f; }
    if (MODE == 2 && id_wt && lane == 0) id_wt[t] = 0.f;
    return;
  }
  float v[MOE_MAX_PER_LANE];
  float s_all[MOE_MAX_PER_LANE];      // MODE 2: the scores themselves (v holds score + correction)
#pragma unroll
  for (int i = 0; i < MOE_MAX_PER_LANE; ++i) {
    const int e = lane + 32 * i;
    v[i] = e < E ? logits[(size_t)t * ld + e] : -INFINITY;
    if (MODE == 1 && e < E) v[i] = 1.0f / (1.0f + expf(-v[i]));
  }
  if (MODE == 2) {
    float mx = -INFINITY;
#pragma unroll
    for (int i = 0; i < MOE_MAX_PER_LANE; ++i) mx = fmaxf(mx, v[i]);
    mx = warp_max(mx);
    float sum = 0.f;
#pragma unroll
    for (int i = 0; i < MOE_MAX_PER_LANE; ++i) {
      s_all[i] = lane + 32 * i < E ? expf(v[i] - mx) : 0.f;
      sum += s_all[i];
    }
    sum = warp_sum(sum);
#pragma unroll
    for (int i = 0; i < MOE_MAX_PER_LANE; ++i) {
      const int e = lane + 32 * i;
      s_all[i] = s_all[i] / sum;
      if (e < E) v[i] = s_all[i] + (correction ? correction[e] : 0.f);
    }
  }
  if (n_groups > 1 && keep < n_groups) {
    // lane g keeps the score of run g (n_groups <= 32): the sum of its two largest scores
    const int per = E / n_groups;
    float mine_g = -INFINITY;
    for (int g = 0; g < n_groups; ++g) {
      float total = 0.f;
      int taken = -1;
      for (int r = 0; r < 2 && r < per; ++r) {
        float best = -INFINITY;
        int best_e = 0x7fffffff;
#pragma unroll
        for (int i = 0; i < MOE_MAX_PER_LANE; ++i) {
          const int e = lane + 32 * i;
          if (e < E && e / per == g && e != taken && (v[i] > best || (v[i] == best && e < best_e))) { best = v[i]; best_e = e; }
        }
        warp_best(best, best_e);
        total += best;
        taken = best_e;
      }
      if (lane == g) mine_g = total;
    }
    uint32_t kept = 0u;
    for (int j = 0; j < keep; ++j) {
      float best = (kept >> lane) & 1u ? -INFINITY : mine_g;
      int best_g = lane < n_groups && !((kept >> lane) & 1u) ? lane : 0x7fffffff;
      warp_best(best, best_g);
      kept |= 1u << best_g;
    }
#pragma unroll
    for (int i = 0; i < MOE_MAX_PER_LANE; ++i) {
      const int e = lane + 32 * i;
      if (e < E && !((kept >> (e / per)) & 1u)) v[i] = -INFINITY;
    }
  }
  float first = 0.f, denom = 0.f, mine = 0.f;      // lane j keeps choice j's weight before the division (top <= 32)
  float id_total = 0.f;
  for (int j = 0; j < top; ++j) {
    float best = -INFINITY;
    int best_e = 0x7fffffff;
#pragma unroll
    for (int i = 0; i < MOE_MAX_PER_LANE; ++i) {
      const int e = lane + 32 * i;
      if (e < E && (v[i] > best || (v[i] == best && e < best_e))) { best = v[i]; best_e = e; }   // (a taken one is -inf: it never wins while a free one is left)
    }
    warp_best(best, best_e);
    if (j == 0) first = best;                        // the largest logit: the softmax's shift
    float ex = MODE == 1 ? best : expf(best - first);
    if (MODE == 2) {                                 // the chosen expert's own score, from the lane that holds it
      float mine_s = 0.f;
#pragma unroll
      for (int i = 0; i < MOE_MAX_PER_LANE; ++i)
        if (lane + 32 * i == best_e) mine_s = s_all[i];
      ex = warp_sum(mine_s) * scale;
      if (best_e >= E - n_identity) {                // an expert that hands its input on
        id_total += ex;
        best_e = -1 - best_e;                        // (marked; written as -1 below)
      }
    }
    denom += ex;
    if (lane == j) mine = ex;
    const int chosen = best_e < 0 ? -1 - best_e : best_e;
    if (lane == 0) idx[(size_t)t * top + j] = best_e < 0 ? -1 : best_e;
    best_e = chosen;
#pragma unroll
    for (int i = 0; i < MOE_MAX_PER_LANE; ++i)
      if (lane + 32 * i == best_e) v[i] = -INFINITY;   // taken
  }
  if (lane < top) wt[(size_t)t * top + lane] = MODE == 2 ? mine : MODE == 1 ? mine / (denom + 1e-20f) : mine / denom;
  if (MODE == 2 && id_wt && lane == 0) id_wt[t] = id_total;
}

// y[t, :] += id_wt[t] * h[t, :] — what the experts that hand their input on add for a token.
template <typename T>
__global__ void __launch_bounds__(256)
moe_identity_add_kernel(const T* __restrict__ h, long ldh, const float* __restrict__ id_wt, float* __restrict__ y, long ldy, int W) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const float w = id_wt[t];
  if (w == 0.f) return;
  for (int c = threadIdx.x; c < W; c += blockDim.x) y[(size_t)t * ldy + c] = fmaf(w, to_f32(h[(size_t)t * ldh + c]), y[(size_t)t * ldy + c]);
}

template <int ACT> __device__ __forceinline__ float moe_act(float g) { return expert_act(g, ACT); }

// A warp's dot product of a shared-memory fp32 vector with one weight row, 16 bytes per lane and load.
template <typename T> struct Vec16;
template <> struct Vec16<__nv_bfloat16> {
  static constexpr int N = 8;
  static __device__ __forceinline__ void load(const __nv_bfloat16* p, float (&v)[8]) {
    const uint4 raw = *reinterpret_cast<const uint4*>(p);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) { const float2 f = __bfloat1622float2(h[i]); v[2 * i] = f.x; v[2 * i + 1] = f.y; }
  }
};
template <> struct Vec16<float> {
  static constexpr int N = 4;
  static __device__ __forceinline__ void load(const float* p, float (&v)[4]) {
    const float4 f = *reinterpret_cast<const float4*>(p);
    v[0] = f.x; v[1] = f.y; v[2] = f.z; v[3] = f.w;
  }
};

// VEC: rows are 16-byte aligned and a multiple of 16 bytes long.  The order of a row's additions is fixed by (K, VEC).
template <typename T, bool VEC>
__device__ __forceinline__ float warp_dot(const float* __restrict__ x_s, const T* __restrict__ row, int K, int lane) {
  float acc = 0.f;
  if (VEC) {
    constexpr int N = Vec16<T>::N;
    for (int i = lane * N; i < K; i += 32 * N) {
      float v[N];
      Vec16<T>::load(row + i, v);
#pragma unroll
      for (int e = 0; e < N; ++e) acc = fmaf(x_s[i + e], v[e], acc);
    }
  } else {
    for (int i = lane; i < K; i += 32) acc = fmaf(x_s[i], to_f32(row[i]), acc);
  }
  return warp_sum(acc);
}

// grid (T * top, ceil(F / 8)); 8 warps, one output f per warp.  wg null: experts without a gate matrix, a = act(Wu h).
template <typename T, int ACT, bool VEC>
__global__ void __launch_bounds__(256)
moe_up_kernel(const T* __restrict__ h, long ldh, const T* __restrict__ wg, const T* __restrict__ wu, int W, int F, int top,
              const int32_t* __restrict__ idx, float* __restrict__ a) {
  extern __shared__ float h_s[];
  pdl_launch_dependents();
  pdl_wait();
  const int item = blockIdx.x, t = item / top;
  const int e = idx[item];
  if (e < 0) return;
  for (int i = threadIdx.x; i < W; i += blockDim.x) h_s[i] = to_f32(h[(size_t)t * ldh + i]);
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int f = blockIdx.y * 8 + warp;
  if (f >= F) return;
  const float u = warp_dot<T, VEC>(h_s, wu + ((size_t)e * F + f) * W, W, lane);
  if (wg == nullptr) {
    if (lane == 0) a[(size_t)item * F + f] = moe_act<ACT>(u);
    return;
  }
  const float g = warp_dot<T, VEC>(h_s, wg + ((size_t)e * F + f) * W, W, lane);
  if (lane == 0) a[(size_t)item * F + f] = moe_act<ACT>(g) * u;
}

// grid (T, ceil(W / 8)); the token's activations [top, F] in shared memory.
template <typename T, bool VEC>
__global__ void __launch_bounds__(256)
moe_down_kernel(const float* __restrict__ a, const T* __restrict__ wd, int W, int F, int top, const int32_t* __restrict__ idx,
                const float* __restrict__ wt, float* __restrict__ y, long ldy, int add) {
  extern __shared__ float a_s[];
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  for (int i = threadIdx.x; i < top * F; i += blockDim.x) a_s[i] = a[(size_t)t * top * F + i];
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int c = blockIdx.y * 8 + warp;
  if (c >= W) return;
  float total = 0.f;
  for (int j = 0; j < top; ++j) {
    const int e = idx[(size_t)t * top + j];
    if (e < 0) continue;
    const float s = warp_dot<T, VEC>(a_s + (size_t)j * F, wd + ((size_t)e * W + c) * F, F, lane);
    total = fmaf(wt[(size_t)t * top + j], s, total);
  }
  if (lane == 0) y[(size_t)t * ldy + c] = add ? y[(size_t)t * ldy + c] + total : total;
}

}  // namespace llmi

using namespace llmi;

// mode 0: softmax over the chosen logits; mode 1: logistic scores normalised over the chosen.  n_groups <= 1 or
// keep >= n_groups: every expert can be chosen.
LLMI_EXPORT int llmi_moe_route(const float* logits, long ld, int E, int top, int mode, int n_groups, int keep,
                               const int32_t* tok_seq, int32_t* idx, float* wt, int n_tokens, const float* correction,
                               float scale, int n_identity, float* id_wt, cudaStream_t stream) {
  if (n_tokens <= 0 || E <= 0 || top <= 0 || top > E || top > 32 || E > 32 * MOE_MAX_PER_LANE) return LLMI_ERR_BAD_SIZE;
  if (n_groups > 1 && (n_groups > 32 || E % n_groups != 0 || keep < 1 || keep * (E / n_groups) < top)) return LLMI_ERR_BAD_SIZE;
  if (n_identity < 0 || n_identity > E || (n_identity > 0 && (mode != 2 || !id_wt))) return LLMI_ERR_BAD_SIZE;
  if (mode == 0)
    return launch_pdl(PDL_SMALL, moe_route_kernel<0>, (n_tokens + 3) / 4, 128, 0, stream, logits, ld, E, top, n_groups, keep, tok_seq,
                      idx, wt, n_tokens, correction, scale, n_identity, id_wt);
  if (mode == 1)
    return launch_pdl(PDL_SMALL, moe_route_kernel<1>, (n_tokens + 3) / 4, 128, 0, stream, logits, ld, E, top, n_groups, keep, tok_seq,
                      idx, wt, n_tokens, correction, scale, n_identity, id_wt);
  if (mode == 2) {
    if (n_groups > 1) return LLMI_ERR_UNSUPPORTED;
    return launch_pdl(PDL_SMALL, moe_route_kernel<2>, (n_tokens + 3) / 4, 128, 0, stream, logits, ld, E, top, n_groups, keep, tok_seq,
                      idx, wt, n_tokens, correction, scale, n_identity, id_wt);
  }
  return LLMI_ERR_UNSUPPORTED;
}

// y [T, ldy] fp32 += id_wt[t] * h[t] (h [T, ldh] in `dtype`).
LLMI_EXPORT int llmi_moe_identity_add(int dtype, const void* h, long ldh, const float* id_wt, float* y, long ldy, int W,
                                      int n_tokens, cudaStream_t stream) {
  if (n_tokens <= 0 || W <= 0) return LLMI_ERR_BAD_SIZE;
  if (dtype == LLMI_DTYPE_F32)
    return launch_pdl(PDL_SMALL, moe_identity_add_kernel<float>, dim3(n_tokens), dim3(256), 0, stream, (const float*)h, ldh, id_wt, y, ldy, W);
  if (dtype == LLMI_DTYPE_BF16)
    return launch_pdl(PDL_SMALL, moe_identity_add_kernel<__nv_bfloat16>, dim3(n_tokens), dim3(256), 0, stream, (const __nv_bfloat16*)h,
                      ldh, id_wt, y, ldy, W);
  return LLMI_ERR_BAD_DTYPE;
}

template <typename T, int ACT, bool VEC>
static int launch_moe_up(const void* h, long ldh, const void* wg, const void* wu, int W, int F, int top, const int32_t* idx, float* a,
                         int n_tokens, cudaStream_t stream) {
  const size_t smem = (size_t)W * 4;
  static PerDevice<size_t> allowed;
  if (smem > 48 * 1024 && allowed.here() < smem) {
    if (cudaFuncSetAttribute(moe_up_kernel<T, ACT, VEC>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
      return LLMI_ERR_BAD_SIZE;
    allowed.here() = smem;
  }
  return launch_pdl(PDL_GEMM, moe_up_kernel<T, ACT, VEC>, dim3(n_tokens * top, (F + 7) / 8), dim3(256), smem, stream, (const T*)h, ldh,
                    (const T*)wg, (const T*)wu, W, F, top, idx, a);
}

template <typename T, bool VEC>
static int launch_moe_down(const float* a, const void* wd, int W, int F, int top, const int32_t* idx, const float* wt, float* y, long ldy,
                           int n_tokens, int add, cudaStream_t stream) {
  const size_t smem = (size_t)top * F * 4;
  static PerDevice<size_t> allowed;
  if (smem > 48 * 1024 && allowed.here() < smem) {
    if (cudaFuncSetAttribute(moe_down_kernel<T, VEC>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
      return LLMI_ERR_BAD_SIZE;
    allowed.here() = smem;
  }
  return launch_pdl(PDL_GEMM, moe_down_kernel<T, VEC>, dim3(n_tokens, (W + 7) / 8), dim3(256), smem, stream, a, (const T*)wd, W, F, top,
                    idx, wt, y, ldy, add);
}

LLMI_EXPORT int llmi_moe_up(int dtype, const void* h, long ldh, const void* wg, const void* wu, int W, int F, int top,
                            const int32_t* idx, float* a, int act, int n_tokens, cudaStream_t stream) {
  if (n_tokens <= 0 || W <= 0 || F <= 0 || top <= 0 || (size_t)W * 4 > 160 * 1024 || (F + 7) / 8 > 65535) return LLMI_ERR_BAD_SIZE;
  if (act < 0 || act > 3) return LLMI_ERR_UNSUPPORTED;
  const int esz = dtype == LLMI_DTYPE_F32 ? 4 : 2;
  const bool vec = ((size_t)W * esz) % 16 == 0 && !((uintptr_t)wg & 15) && !((uintptr_t)wu & 15);
#define LLMI_UP(T, ACT) \
  return vec ? launch_moe_up<T, ACT, true>(h, ldh, wg, wu, W, F, top, idx, a, n_tokens, stream) \
             : launch_moe_up<T, ACT, false>(h, ldh, wg, wu, W, F, top, idx, a, n_tokens, stream)
  if (dtype == LLMI_DTYPE_F32) {
    if (act == 0) LLMI_UP(float, 0); else if (act == 1) LLMI_UP(float, 1); else if (act == 2) LLMI_UP(float, 2); else LLMI_UP(float, 3);
  }
  if (dtype == LLMI_DTYPE_BF16) {
    if (act == 0) LLMI_UP(__nv_bfloat16, 0); else if (act == 1) LLMI_UP(__nv_bfloat16, 1);
    else if (act == 2) LLMI_UP(__nv_bfloat16, 2); else LLMI_UP(__nv_bfloat16, 3);
  }
#undef LLMI_UP
  return LLMI_ERR_BAD_DTYPE;
}

LLMI_EXPORT int llmi_moe_down(int dtype, const float* a, const void* wd, int W, int F, int top, const int32_t* idx,
                              const float* wt, float* y, long ldy, int n_tokens, int add, cudaStream_t stream) {
  if (n_tokens <= 0 || W <= 0 || F <= 0 || top <= 0 || (size_t)top * F * 4 > 160 * 1024 || (W + 7) / 8 > 65535) return LLMI_ERR_BAD_SIZE;
  const int esz = dtype == LLMI_DTYPE_F32 ? 4 : 2;
  const bool vec = ((size_t)F * esz) % 16 == 0 && !((uintptr_t)wd & 15);
  if (dtype == LLMI_DTYPE_F32)
    return vec ? launch_moe_down<float, true>(a, wd, W, F, top, idx, wt, y, ldy, n_tokens, add, stream)
               : launch_moe_down<float, false>(a, wd, W, F, top, idx, wt, y, ldy, n_tokens, add, stream);
  if (dtype == LLMI_DTYPE_BF16)
    return vec ? launch_moe_down<__nv_bfloat16, true>(a, wd, W, F, top, idx, wt, y, ldy, n_tokens, add, stream)
               : launch_moe_down<__nv_bfloat16, false>(a, wd, W, F, top, idx, wt, y, ldy, n_tokens, add, stream);
  return LLMI_ERR_BAD_DTYPE;
}
