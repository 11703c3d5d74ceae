// A short causal convolution over time on every channel of a step's rows, added to its own input:
//     y[t, c] = h[t, c] + sum_{j < K} w[j, c] * h[t - (K-1) + j, c]          (zeros before a sequence's start)
// The K-1 rows ahead of a step's first token come from the sequence's state (`carry`, fp32, [K-1][C] per slot:
// the inputs at positions p0-(K-1) .. p0-1), which a second kernel brings up to date after the step.  The sum is
// fp32, taps in the order oldest first, so a position's result does not depend on how its sequence was cut.
//
//   llmi_conv_add     one thread per (token, channel)
//   llmi_conv_carry   one thread per (sequence, channel): the inputs of the last K-1 positions after this step,
//                     from the step's own rows or, where the step brought fewer, from what the state held
//   llmi_norm_conv_token   a step of single tokens: the norm ahead, the convolution and the state's update in one
#include "common.cuh"

namespace llmi {

constexpr int CONV_MAX_TAPS = 16;

template <typename T>
__global__ void __launch_bounds__(128)
conv_add_kernel(const T* __restrict__ h, long ldh, const float* __restrict__ w, const float* __restrict__ carry_all,
                long carry_stride, const int32_t* __restrict__ tok_seq, const int32_t* __restrict__ tok_pos,
                const int32_t* __restrict__ seq_q_start, const int32_t* __restrict__ seq_slot, T* __restrict__ y, long ldy,
                int C, int K, int add_input) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const int c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= C) return;
  const int seq = tok_seq[t];
  if (seq < 0) {
    y[(size_t)t * ldy + c] = from_f32<T>(0.f);
    return;
  }
  const int slot = seq_slot[seq];
  const int pos = tok_pos[t], r0 = seq_q_start[seq];
  const int p0 = pos - (t - r0);                              // position of this sequence's first row of the step
  const float* carry = carry_all + (size_t)(slot < 0 ? 0 : slot) * carry_stride;
  const float own = add_input ? to_f32(h[(size_t)t * ldh + c]) : 0.f;
  float acc = 0.f;
  for (int j = 0; j < K; ++j) {                               // oldest tap first
    const int p = pos - (K - 1) + j;
    if (p < 0) continue;
    const float x = p >= p0 ? to_f32(h[(size_t)(r0 + (p - p0)) * ldh + c]) : carry[(size_t)(p - (p0 - (K - 1))) * C + c];
    acc = fmaf(x, w[(size_t)j * C + c], acc);
  }
  y[(size_t)t * ldy + c] = from_f32<T>(own + acc);
}

// The same for bf16 rows whose channels come in whole groups of eight (16-byte accesses): one thread per (token, eight
// channels); the sums and their order are those of the kernel above.
__global__ void __launch_bounds__(128)
conv_add_vec8_kernel(const __nv_bfloat16* __restrict__ h, long ldh, const float* __restrict__ w, const float* __restrict__ carry_all,
                     long carry_stride, const int32_t* __restrict__ tok_seq, const int32_t* __restrict__ tok_pos,
                     const int32_t* __restrict__ seq_q_start, const int32_t* __restrict__ seq_slot, __nv_bfloat16* __restrict__ y,
                     long ldy, int C, int K) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const int c = (blockIdx.y * blockDim.x + threadIdx.x) * 8;
  if (c >= C) return;
  const int seq = tok_seq[t];
  if (seq < 0) {
    *reinterpret_cast<uint4*>(y + (size_t)t * ldy + c) = make_uint4(0u, 0u, 0u, 0u);
    return;
  }
  const int slot = seq_slot[seq];
  const int pos = tok_pos[t], r0 = seq_q_start[seq];
  const int p0 = pos - (t - r0);
  const float* carry = carry_all + (size_t)(slot < 0 ? 0 : slot) * carry_stride;
  float acc[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) acc[e] = 0.f;
  for (int j = 0; j < K; ++j) {
    const int p = pos - (K - 1) + j;
    if (p < 0) continue;
    float x[8];
    if (p >= p0) {
      const uint4 raw = *reinterpret_cast<const uint4*>(h + (size_t)(r0 + (p - p0)) * ldh + c);
      const __nv_bfloat162* pr = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 f = __bfloat1622float2(pr[e]);
        x[2 * e] = f.x;
        x[2 * e + 1] = f.y;
      }
    } else {
      const float* cr = carry + (size_t)(p - (p0 - (K - 1))) * C + c;
#pragma unroll
      for (int e = 0; e < 8; ++e) x[e] = cr[e];
    }
    const float4 w0 = *reinterpret_cast<const float4*>(w + (size_t)j * C + c), w1 = *reinterpret_cast<const float4*>(w + (size_t)j * C + c + 4);
    const float we[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[e] = fmaf(x[e], we[e], acc[e]);
  }
  const uint4 raw = *reinterpret_cast<const uint4*>(h + (size_t)t * ldh + c);
  const __nv_bfloat162* pr = reinterpret_cast<const __nv_bfloat162*>(&raw);
  uint4 outv;
  __nv_bfloat162* po = reinterpret_cast<__nv_bfloat162*>(&outv);
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    const float2 f = __bfloat1622float2(pr[e]);
    po[e] = __floats2bfloat162_rn(f.x + acc[2 * e], f.y + acc[2 * e + 1]);
  }
  *reinterpret_cast<uint4*>(y + (size_t)t * ldy + c) = outv;
}

// The convolution alone (the input itself is not added) on fp32 rows whose channels come in whole groups of four
// (16-byte accesses): one thread per (token, four channels); the sums and their order are those of conv_add_kernel.
__global__ void __launch_bounds__(128)
conv_vec4_kernel(const float* __restrict__ h, long ldh, const float* __restrict__ w, const float* __restrict__ carry_all,
                 long carry_stride, const int32_t* __restrict__ tok_seq, const int32_t* __restrict__ tok_pos,
                 const int32_t* __restrict__ seq_q_start, const int32_t* __restrict__ seq_slot, float* __restrict__ y, long ldy,
                 int C, int K) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const int c = (blockIdx.y * blockDim.x + threadIdx.x) * 4;
  if (c >= C) return;
  const int seq = tok_seq[t];
  if (seq < 0) {
    *reinterpret_cast<float4*>(y + (size_t)t * ldy + c) = make_float4(0.f, 0.f, 0.f, 0.f);
    return;
  }
  const int slot = seq_slot[seq];
  const int pos = tok_pos[t], r0 = seq_q_start[seq];
  const int p0 = pos - (t - r0);
  const float* carry = carry_all + (size_t)(slot < 0 ? 0 : slot) * carry_stride;
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int j = 0; j < K; ++j) {                               // oldest tap first
    const int p = pos - (K - 1) + j;
    if (p < 0) continue;
    const float4 x = p >= p0 ? *reinterpret_cast<const float4*>(h + (size_t)(r0 + (p - p0)) * ldh + c)
                             : *reinterpret_cast<const float4*>(carry + (size_t)(p - (p0 - (K - 1))) * C + c);
    const float4 wj = *reinterpret_cast<const float4*>(w + (size_t)j * C + c);
    acc.x = fmaf(x.x, wj.x, acc.x);
    acc.y = fmaf(x.y, wj.y, acc.y);
    acc.z = fmaf(x.z, wj.z, acc.z);
    acc.w = fmaf(x.w, wj.w, acc.w);
  }
  *reinterpret_cast<float4*>(y + (size_t)t * ldy + c) = acc;
}

template <typename T>
__global__ void __launch_bounds__(128)
conv_carry_kernel(const T* __restrict__ h, long ldh, float* __restrict__ carry_all, long carry_stride,
                  const int32_t* __restrict__ seq_q_start, const int32_t* __restrict__ seq_kv_len,
                  const int32_t* __restrict__ seq_slot, int C, int K) {
  pdl_launch_dependents();
  pdl_wait();
  const int seq = blockIdx.y;
  const int slot = seq_slot[seq];
  if (slot < 0) return;
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  const int r0 = seq_q_start[seq], n = seq_q_start[seq + 1] - r0, L = seq_kv_len[seq];
  if (n <= 0) return;
  const int p0 = L - n;
  float* carry = carry_all + (size_t)slot * carry_stride;
  float keep[CONV_MAX_TAPS];
  for (int j = 0; j < K - 1; ++j) {
    const int p = L - (K - 1) + j;
    keep[j] = p < 0 ? 0.f
                    : (p >= p0 ? to_f32(h[(size_t)(r0 + (p - p0)) * ldh + c]) : carry[(size_t)(p - (p0 - (K - 1))) * C + c]);
  }
  for (int j = 0; j < K - 1; ++j) carry[(size_t)j * C + c] = keep[j];
}

// A step in which every sequence brings ONE token: the RMS norm ahead of the convolution, the convolution and the
// state's update in one kernel, one thread per (token, channel).  h = T(weight * (x * rsqrt(mean(x^2) + eps))) is rounded to the
// compute type as the norm kernel rounds it, the taps are added oldest first as above, and the thread that owns a
// channel reads its state entries before it writes them: the results are those of the three kernels.
template <typename T>
__global__ void __launch_bounds__(256)
norm_conv_token_kernel(const float* __restrict__ x, const float* __restrict__ norm_w, float eps, const float* __restrict__ w,
                       float* carry_all, long carry_stride, const int32_t* __restrict__ tok_seq,
                       const int32_t* __restrict__ seq_slot, T* __restrict__ y, long ldy, int C, int K, int write_state) {
  __shared__ float scratch[32];
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const int c = blockIdx.y * blockDim.x + threadIdx.x;       // my channel; every block of a token sums the whole row itself
  const int seq = tok_seq[t];
  const int slot = seq < 0 ? -1 : seq_slot[seq];
  if (slot < 0) {
    if (c < C) y[(size_t)t * ldy + c] = from_f32<T>(0.f);
    return;
  }
  const float* xr = x + (size_t)t * C;
  float ss = 0.f;
  for (int i = threadIdx.x; i < C; i += blockDim.x) ss = fmaf(xr[i], xr[i], ss);
  ss = block_sum(ss, scratch);
  if (c >= C) return;
  const float scale = 1.0f / sqrtf(ss / (float)C + eps);
  float* carry = carry_all + (size_t)slot * carry_stride;
  float old[CONV_MAX_TAPS];
#pragma unroll
  for (int j = 0; j < CONV_MAX_TAPS - 1; ++j)
    if (j < K - 1) old[j] = carry[(size_t)j * C + c];          // all of my state first: independent loads, and read before written
  const float h = to_f32(from_f32<T>(norm_w[c] * (xr[c] * scale)));
  float acc = 0.f;
#pragma unroll
  for (int j = 0; j < CONV_MAX_TAPS - 1; ++j)
    if (j < K - 1) acc = fmaf(old[j], w[(size_t)j * C + c], acc);
  acc = fmaf(h, w[(size_t)(K - 1) * C + c], acc);
  y[(size_t)t * ldy + c] = from_f32<T>(h + acc);
  if (write_state && K > 1) {
#pragma unroll
    for (int j = 1; j < CONV_MAX_TAPS - 1; ++j)
      if (j < K - 1) carry[(size_t)(j - 1) * C + c] = old[j];
    carry[(size_t)(K - 2) * C + c] = h;
  }
}

// A step in which every sequence brings ONE token, fp32 rows, the convolution alone (the input itself is not added)
// and the state's update in one kernel, one thread per (token, channel): the taps are added oldest first as in
// conv_add_kernel, and the thread that owns a channel reads its state entries before it writes them — the results of
// llmi_conv_add (without the input) + llmi_conv_carry.
__global__ void __launch_bounds__(256)
conv_token_kernel(const float* __restrict__ h, long ldh, const float* __restrict__ w, float* carry_all, long carry_stride,
                  const int32_t* __restrict__ tok_seq, const int32_t* __restrict__ seq_slot, float* __restrict__ y, long ldy, int C,
                  int K, int write_state) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const int c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= C) return;
  const int seq = tok_seq[t];
  const int slot = seq < 0 ? -1 : seq_slot[seq];
  if (slot < 0) {
    y[(size_t)t * ldy + c] = 0.f;
    return;
  }
  float* carry = carry_all + (size_t)slot * carry_stride;
  float old[CONV_MAX_TAPS];
#pragma unroll
  for (int j = 0; j < CONV_MAX_TAPS - 1; ++j)
    if (j < K - 1) old[j] = carry[(size_t)j * C + c];          // all of my state first: independent loads, and read before written
  const float x = h[(size_t)t * ldh + c];
  float acc = 0.f;
#pragma unroll
  for (int j = 0; j < CONV_MAX_TAPS - 1; ++j)
    if (j < K - 1) acc = fmaf(old[j], w[(size_t)j * C + c], acc);
  acc = fmaf(x, w[(size_t)(K - 1) * C + c], acc);
  y[(size_t)t * ldy + c] = acc;
  if (write_state && K > 1) {
#pragma unroll
    for (int j = 1; j < CONV_MAX_TAPS - 1; ++j)
      if (j < K - 1) carry[(size_t)(j - 1) * C + c] = old[j];
    carry[(size_t)(K - 2) * C + c] = x;
  }
}

}  // namespace llmi

using namespace llmi;

// For a step of single tokens: y [T, C] fp32 = conv(h) (the input itself not added) of the fp32 rows h, and the state
// brought up to date.  A state entry before a sequence's start is zero (a slot's state is cleared when it is handed
// out), so the taps that reach before position 0 add nothing.
LLMI_EXPORT int llmi_conv_token(const float* h, long ldh, const float* w, float* carry, long carry_stride, const int32_t* tok_seq,
                                const int32_t* seq_slot, float* y, long ldy, int n_tokens, int C, int K, int write_state,
                                cudaStream_t stream) {
  if (n_tokens <= 0 || C <= 0 || K < 1 || K > CONV_MAX_TAPS) return LLMI_ERR_BAD_SIZE;
  const int threads = C >= 1024 ? 256 : (C >= 256 ? 128 : 64);
  const dim3 grid(n_tokens, (C + threads - 1) / threads);
  if (grid.y > 65535) return LLMI_ERR_BAD_SIZE;
  return launch_pdl(PDL_SMALL, conv_token_kernel, grid, dim3(threads), 0, stream, h, ldh, w, carry, carry_stride, tok_seq, seq_slot,
                    y, ldy, C, K, write_state);
}

// For a step of single tokens: y [T, C] (type `dtype`) = h + conv(h) with h the RMS norm of the fp32 rows x [T, C]
// (contiguous), and the state brought up to date.
LLMI_EXPORT int llmi_norm_conv_token(int dtype, const float* x, const float* norm_w, float eps, const float* w, float* carry,
                                     long carry_stride, const int32_t* tok_seq, const int32_t* seq_slot, void* y, long ldy,
                                     int n_tokens, int C, int K, int write_state, cudaStream_t stream) {
  if (n_tokens <= 0 || C <= 0 || K < 1 || K > CONV_MAX_TAPS) return LLMI_ERR_BAD_SIZE;
  const int threads = C >= 1024 ? 256 : (C >= 256 ? 128 : 64);
  const dim3 grid(n_tokens, (C + threads - 1) / threads);
  if (grid.y > 65535) return LLMI_ERR_BAD_SIZE;
  if (dtype == LLMI_DTYPE_F32)
    return launch_pdl(PDL_SMALL, norm_conv_token_kernel<float>, grid, dim3(threads), 0, stream, x, norm_w, eps, w, carry,
                      carry_stride, tok_seq, seq_slot, (float*)y, ldy, C, K, write_state);
  if (dtype == LLMI_DTYPE_BF16)
    return launch_pdl(PDL_SMALL, norm_conv_token_kernel<__nv_bfloat16>, grid, dim3(threads), 0, stream, x, norm_w, eps, w,
                      carry, carry_stride, tok_seq, seq_slot, (__nv_bfloat16*)y, ldy, C, K, write_state);
  return LLMI_ERR_BAD_DTYPE;
}

// y = h + conv(h), or conv(h) alone without `add_input`; h, y [T, C] in the type `dtype`; w fp32 [K, C] (tap-major); carry fp32 [slots, carry_stride >= (K-1)*C].
LLMI_EXPORT int llmi_conv_add(int dtype, const void* h, long ldh, const float* w, const float* carry, long carry_stride,
                              const int32_t* tok_seq, const int32_t* tok_pos, const int32_t* seq_q_start,
                              const int32_t* seq_slot, void* y, long ldy, int n_tokens, int C, int K, int add_input,
                              cudaStream_t stream) {
  if (n_tokens <= 0 || C <= 0 || (C + 127) / 128 > 65535 || K < 1 || K > CONV_MAX_TAPS) return LLMI_ERR_BAD_SIZE;
  const dim3 grid(n_tokens, (C + 127) / 128);
  if (dtype == LLMI_DTYPE_F32 && !add_input && C % 4 == 0 && ldh % 4 == 0 && ldy % 4 == 0 && carry_stride % 4 == 0 &&
      !((uintptr_t)h & 15) && !((uintptr_t)y & 15) && !((uintptr_t)w & 15) && !((uintptr_t)carry & 15)) {
    const int threads = C / 4 >= 128 ? 128 : ((C / 4 + 31) / 32) * 32;
    return launch_pdl(PDL_SMALL, conv_vec4_kernel, dim3(n_tokens, (C / 4 + threads - 1) / threads), dim3(threads), 0, stream,
                      (const float*)h, ldh, w, carry, carry_stride, tok_seq, tok_pos, seq_q_start, seq_slot, (float*)y, ldy, C, K);
  }
  if (dtype == LLMI_DTYPE_F32)
    return launch_pdl(PDL_SMALL, conv_add_kernel<float>, grid, dim3(128), 0, stream, (const float*)h, ldh, w, carry, carry_stride,
                      tok_seq, tok_pos, seq_q_start, seq_slot, (float*)y, ldy, C, K, add_input);
  if (dtype == LLMI_DTYPE_BF16) {
    if (add_input && C % 8 == 0 && ldh % 8 == 0 && ldy % 8 == 0 && !((uintptr_t)h & 15) && !((uintptr_t)y & 15) && !((uintptr_t)w & 15)) {
      const int threads = C / 8 >= 128 ? 128 : ((C / 8 + 31) / 32) * 32;
      return launch_pdl(PDL_SMALL, conv_add_vec8_kernel, dim3(n_tokens, (C / 8 + threads - 1) / threads), dim3(threads), 0, stream,
                        (const __nv_bfloat16*)h, ldh, w, carry, carry_stride, tok_seq, tok_pos, seq_q_start, seq_slot,
                        (__nv_bfloat16*)y, ldy, C, K);
    }
    return launch_pdl(PDL_SMALL, conv_add_kernel<__nv_bfloat16>, grid, dim3(128), 0, stream, (const __nv_bfloat16*)h, ldh, w, carry,
                      carry_stride, tok_seq, tok_pos, seq_q_start, seq_slot, (__nv_bfloat16*)y, ldy, C, K, add_input);
  }
  return LLMI_ERR_BAD_DTYPE;
}

LLMI_EXPORT int llmi_conv_carry(int dtype, const void* h, long ldh, float* carry, long carry_stride, const int32_t* seq_q_start,
                                const int32_t* seq_kv_len, const int32_t* seq_slot, int n_seqs, int C, int K,
                                cudaStream_t stream) {
  if (n_seqs <= 0 || n_seqs > 65535 || C <= 0 || K < 1 || K > CONV_MAX_TAPS) return LLMI_ERR_BAD_SIZE;
  if (K == 1) return LLMI_OK;
  const dim3 grid((C + 127) / 128, n_seqs);
  if (dtype == LLMI_DTYPE_F32)
    return launch_pdl(PDL_SMALL, conv_carry_kernel<float>, grid, dim3(128), 0, stream, (const float*)h, ldh, carry, carry_stride,
                      seq_q_start, seq_kv_len, seq_slot, C, K);
  if (dtype == LLMI_DTYPE_BF16)
    return launch_pdl(PDL_SMALL, conv_carry_kernel<__nv_bfloat16>, grid, dim3(128), 0, stream, (const __nv_bfloat16*)h, ldh, carry,
                      carry_stride, seq_q_start, seq_kv_len, seq_slot, C, K);
  return LLMI_ERR_BAD_DTYPE;
}
