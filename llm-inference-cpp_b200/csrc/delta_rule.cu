// The gated delta rule: a recurrent mixer whose per-head state S [D, Dv] is a fast-weight matrix,
//     S <- g S;   u = beta (v - Sᵀ k);   S <- S + k uᵀ;   o = Sᵀ q        (in this order, per token)
// with q, k unit vectors (q also times D^-1/2), a decay g in (0, 1) and a write strength beta in (0, 1).
// q, k, v first pass a short causal convolution over time (per channel, no bias) and silu.  The state of a
// sequence is S (fp32) and the last taps-1 inputs of the convolution (fp32); both live in the cache's state slab,
// one row per slot:  [ S: H*Dv*D | conv: (taps-1) * Nc ],  Nc = 2*Hk*D + H*Dv channels.  S is kept column by column
// ([head][column j][entry d]): the threads that share a column read and write neighbouring words.
//
// Everything here is fp32 arithmetic.  Kernels, in the order of a step:
//   llmi_delta_prepare      per (token, piece): convolution + silu, unit norms, beta, decay (parallel over tokens)
//   llmi_delta_conv_carry   per sequence: the convolution's inputs that the next step needs (after prepare)
//   llmi_delta_recurrence   per (sequence, head, slice of columns): the recurrence over the step's tokens
//   llmi_delta_finish       per (token, head): o / rms(o) * w * act(gate) in the compute type (parallel over tokens)
// The input `proj` is one fp32 row per token: [ q (Hk*D) | k (Hk*D) | v (H*Dv) | b (H) | a (H) | gate (H*Dv) ].
// The recurrence treats a column of S alone, and a step only continues what the slab holds: the result does not
// depend on how a prompt was cut or on what else is in the batch.
#include <math.h>

#include "common.cuh"

namespace llmi {

constexpr int DELTA_MAX_TAPS = 16;

struct DeltaDims {
  int H, Hk, D, Dv, taps;
  __host__ __device__ int n_qk() const { return 2 * Hk * D; }
  __host__ __device__ int n_conv() const { return 2 * Hk * D + H * Dv; }
  __host__ __device__ long state_floats() const { return (long)H * D * Dv + (long)(taps - 1) * n_conv(); }
  __host__ __device__ long conv_offset() const { return (long)H * D * Dv; }
};

__device__ __forceinline__ float silu_f(float z) { return z / (1.0f + expf(-z)); }
__device__ __forceinline__ float softplus_f(float z) { return z > 20.f ? z : log1pf(expf(z)); }

// One block per (token, piece).  Pieces 0 .. 2 Hk - 1: one head of q or k (convolution, silu, unit norm); the pieces
// behind them: 256 channels of v each (convolution, silu); the last piece also makes beta and decay of every head.
// prep: fp32 [T, Nc + 2H]: [ q^ | k^ | v | beta | decay ].
constexpr int DELTA_V_PIECE = 256;

__device__ __forceinline__ float delta_conv_one(const float* __restrict__ proj, long ld, const float* __restrict__ carry,
                                                const float* __restrict__ conv_w, int ch, int Nc, int K, int pos, int p0, int r0) {
  float acc = 0.f;
  for (int d = K - 1; d >= 0; --d) {                     // oldest tap first
    const int p = pos - d;
    if (p < 0) continue;
    const float x = p >= p0 ? proj[(size_t)(r0 + (p - p0)) * ld + ch] : carry[(size_t)(p - (p0 - (K - 1))) * Nc + ch];
    acc = fmaf(x, conv_w[(size_t)ch * K + (K - 1 - d)], acc);
  }
  return silu_f(acc);
}

__global__ void __launch_bounds__(256)
delta_prepare_kernel(const float* __restrict__ proj, long ld, DeltaDims m, const float* __restrict__ conv_w,
                     const float* __restrict__ a_log, const float* __restrict__ dt_bias, const float* __restrict__ state,
                     const int32_t* __restrict__ tok_seq, const int32_t* __restrict__ tok_pos,
                     const int32_t* __restrict__ seq_q_start, const int32_t* __restrict__ seq_slot,
                     float* __restrict__ prep, long ldp) {
  __shared__ float scratch[32];
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x, piece = blockIdx.y;
  const int seq = tok_seq[t];
  if (seq < 0) return;
  const int slot = seq_slot[seq];
  if (slot < 0) return;
  const int pos = tok_pos[t], r0 = seq_q_start[seq];
  const int p0 = pos - (t - r0);                         // position of the step's first token of this sequence
  const int K = m.taps, Nc = m.n_conv(), Nqk = m.n_qk();
  const float* carry = state + (size_t)slot * m.state_floats() + m.conv_offset();   // [K-1][Nc]: positions p0-(K-1) .. p0-1
  float* out = prep + (size_t)t * ldp;
  if (piece < 2 * m.Hk) {
    // a head of q (pieces 0 .. Hk-1) or of k: its D channels, then the unit norm over them
    const int base = piece * m.D;
    float ss = 0.f;
    for (int d = threadIdx.x; d < m.D; d += blockDim.x) {
      const float y = delta_conv_one(proj, ld, carry, conv_w, base + d, Nc, K, pos, p0, r0);
      out[base + d] = y;                                 // (kept here until the scale is known; the same thread comes back)
      ss = fmaf(y, y, ss);
    }
    ss = block_sum(ss, scratch);
    float sc = 1.0f / sqrtf(ss + 1e-6f);
    if (piece < m.Hk) sc *= 1.0f / sqrtf((float)m.D);
    for (int d = threadIdx.x; d < m.D; d += blockDim.x) out[base + d] *= sc;
    return;
  }
  const int vp = piece - 2 * m.Hk, n_v = m.H * m.Dv;
  for (int c = vp * DELTA_V_PIECE + threadIdx.x; c < min(n_v, (vp + 1) * DELTA_V_PIECE); c += blockDim.x)
    out[Nqk + c] = delta_conv_one(proj, ld, carry, conv_w, Nqk + c, Nc, K, pos, p0, r0);
  if (piece == (int)gridDim.y - 1) {
    const float* row = proj + (size_t)t * ld;
    for (int h = threadIdx.x; h < m.H; h += blockDim.x) {
      const float b = row[Nc + h], a = row[Nc + m.H + h];
      out[Nc + h] = 1.0f / (1.0f + expf(-b));
      out[Nc + m.H + h] = expf(-expf(a_log[h]) * softplus_f(a + dt_bias[h]));
    }
  }
}

// One thread per (sequence, channel): the inputs of the last taps-1 positions after this step, from the step's own
// rows or, where the step brought fewer, from what the slab held.
__global__ void __launch_bounds__(128)
delta_conv_carry_kernel(const float* __restrict__ proj, long ld, DeltaDims m, float* __restrict__ state,
                        const int32_t* __restrict__ seq_q_start, const int32_t* __restrict__ seq_kv_len,
                        const int32_t* __restrict__ seq_slot, int n_seqs) {
  pdl_launch_dependents();
  pdl_wait();
  const int seq = blockIdx.y;
  const int slot = seq_slot[seq];
  if (slot < 0) return;
  const int ch = blockIdx.x * blockDim.x + threadIdx.x;
  const int Nc = m.n_conv(), K = m.taps;
  if (ch >= Nc || K <= 1) return;
  const int r0 = seq_q_start[seq], n = seq_q_start[seq + 1] - r0, L = seq_kv_len[seq];
  if (n <= 0) return;
  const int p0 = L - n;
  float* carry = state + (size_t)slot * m.state_floats() + m.conv_offset();
  float keep[DELTA_MAX_TAPS];
  for (int j = 0; j < K - 1; ++j) {
    const int p = L - (K - 1) + j;
    keep[j] = p < 0 ? 0.f : (p >= p0 ? proj[(size_t)(r0 + (p - p0)) * ld + ch] : carry[(size_t)(p - (p0 - (K - 1))) * Nc + ch]);
  }
  for (int j = 0; j < K - 1; ++j) carry[(size_t)j * Nc + ch] = keep[j];
}

// One block per (head, sequence), one thread per column j of S.  DREG > 0: the column (D = DREG entries) lives in
// registers; DREG == 0: any D, the column lives in shared memory (S_s[d][j]: no two threads share a bank).
// k and q of the next token are fetched while the current one is computed (two buffers, one barrier per token).
template <int DREG>
__global__ void __launch_bounds__(1024)
delta_recurrence_kernel(const float* __restrict__ prep, long ldp, DeltaDims m, float* __restrict__ state,
                        const int32_t* __restrict__ seq_q_start, const int32_t* __restrict__ seq_slot,
                        float* __restrict__ o_raw, long ldo, int write_state) {
  extern __shared__ float sm[];
  pdl_wait();
  pdl_launch_dependents();
  const int h = blockIdx.x, seq = blockIdx.y;
  const int slot = seq_slot[seq];
  if (slot < 0) return;
  const int r0 = seq_q_start[seq], n = seq_q_start[seq + 1] - r0;
  if (n <= 0) return;
  const int D = DREG > 0 ? DREG : m.D, Dv = m.Dv;
  const int cols = blockDim.x;                               // Dv rounded up to whole warps
  const int j = threadIdx.x;
  const bool live = j < Dv;
  float* kq = sm;                                            // [2][2*D]: k then q of a token
  float* S_s = sm + 4 * D;                                   // [D][cols] (DREG == 0 only)
  const int kh = h / (m.H / m.Hk);
  float* S_g = state + (size_t)slot * m.state_floats() + (size_t)h * D * Dv;
  float S_r[DREG > 0 ? DREG : 1];
  if (live) {
    if (DREG > 0) {
#pragma unroll
      for (int d = 0; d < DREG; ++d) S_r[d] = S_g[(size_t)j * D + d];
    } else {
      for (int d = 0; d < D; ++d) S_s[(size_t)d * cols + j] = S_g[(size_t)j * D + d];
    }
  }
  const int Nc = m.n_conv();
  auto fetch = [&](int i, int buf) {
    const float* row = prep + (size_t)(r0 + i) * ldp;
    for (int d = threadIdx.x; d < 2 * D; d += blockDim.x)
      kq[buf * 2 * D + d] = d < D ? row[(size_t)m.Hk * D + (size_t)kh * D + d] : row[(size_t)kh * D + (d - D)];
  };
  fetch(0, 0);
  for (int i = 0; i < n; ++i) {
    __syncthreads();                                         // buffer i&1 is filled; the other one is read out
    if (i + 1 < n) fetch(i + 1, (i + 1) & 1);
    if (!live) continue;
    const float* row = prep + (size_t)(r0 + i) * ldp;
    const float v = row[(size_t)m.n_qk() + (size_t)h * Dv + j];
    const float beta = row[Nc + h], g = row[Nc + m.H + h];
    const float* k = kq + (i & 1) * 2 * D;
    const float* q = k + D;
    float sk = 0.f;
    if (DREG > 0) {
#pragma unroll
      for (int d = 0; d < DREG; ++d) sk = fmaf(S_r[d], k[d], sk);
    } else {
      for (int d = 0; d < D; ++d) sk = fmaf(S_s[(size_t)d * cols + j], k[d], sk);
    }
    const float u = beta * (v - g * sk);                     // (g S)ᵀ k = g (Sᵀ k)
    float o = 0.f;
    if (DREG > 0) {
#pragma unroll
      for (int d = 0; d < DREG; ++d) {
        const float s = fmaf(k[d], u, g * S_r[d]);
        S_r[d] = s;
        o = fmaf(s, q[d], o);
      }
    } else {
      for (int d = 0; d < D; ++d) {
        const float s = fmaf(k[d], u, g * S_s[(size_t)d * cols + j]);
        S_s[(size_t)d * cols + j] = s;
        o = fmaf(s, q[d], o);
      }
    }
    o_raw[(size_t)(r0 + i) * ldo + (size_t)h * Dv + j] = o;
  }
  if (live && write_state) {
    if (DREG > 0) {
#pragma unroll
      for (int d = 0; d < DREG; ++d) S_g[(size_t)j * D + d] = S_r[d];
    } else {
      for (int d = 0; d < D; ++d) S_g[(size_t)j * D + d] = S_s[(size_t)d * cols + j];
    }
  }
}

// The form for D = 32, 64, 128 and Dv a multiple of 16.  A thread holds TWO neighbouring columns of S and a
// sixteenth of their entries (lane `sub` of sixteen: d = 64 i + 4 sub + 0..3, while d < D), in registers; partial sums
// over d are joined by four shuffles.  The recurrence is a chain over the tokens — the time of a prompt is tokens x
// (time of one token), and a token costs one warp's instructions (each warp has a scheduler to itself) — so the
// work of a token is spread thin: 16 columns a warp.  Columns are independent: a head's columns are cut into slices
// of 32 (or 16) and every slice is a block of its own (blockIdx.z).
//
// What a token needs — k, q of the head's key head, the slice's v, beta, g — is copied into a ring of DELTA_RING
// entries DELTA_RING - 1 tokens ahead (cp.async, 16 bytes a copy, no registers in between), so that no load's latency
// lies on the chain from token to token; one barrier per token.
constexpr int DELTA_RING = 8;

__device__ __forceinline__ void cp_async4(void* dst, const void* src) {
  const uint32_t d = (uint32_t)__cvta_generic_to_shared(dst);
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(d), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async16_ca(void* dst, const void* src) {
  const uint32_t d = (uint32_t)__cvta_generic_to_shared(dst);
  asm volatile("cp.async.ca.shared.global [%0], [%1], 16;" ::"r"(d), "l"(src) : "memory");
}

template <int D>
__global__ void __launch_bounds__(256)
delta_recurrence_quad_kernel(const float* __restrict__ prep, long ldp, DeltaDims m, float* __restrict__ state,
                             const int32_t* __restrict__ seq_q_start, const int32_t* __restrict__ seq_slot,
                             float* __restrict__ o_raw, long ldo, int write_state) {
  extern __shared__ __align__(16) float sm[];
  pdl_wait();
  pdl_launch_dependents();
  const int h = blockIdx.x, seq = blockIdx.y;
  const int slot = seq_slot[seq];
  if (slot < 0) return;
  const int r0 = seq_q_start[seq], n = seq_q_start[seq + 1] - r0;
  if (n <= 0) return;
  constexpr int NI = (D + 63) / 64;                          // chunks of four entries per lane (D = 32: lanes 8..15 hold none)
  const int Dv = m.Dv;
  const int CB = blockDim.x >> 3;                            // columns of this block's slice (the launcher gives 8 CB threads)
  const int cg = threadIdx.x >> 4, sub = threadIdx.x & 15;   // my columns: col0, col0 + 1
  const int col0 = blockIdx.z * CB + 2 * cg;
  const bool holds = 4 * sub < D;                            // (D = 32 only: half of the lanes carry zeros)
  const int kh = h / (m.H / m.Hk);
  float* S_g = state + (size_t)slot * m.state_floats() + (size_t)h * D * Dv + (size_t)col0 * D;    // [column][entry]
  float2 S_r[NI][4];                                         // [chunk][entry of the chunk] . (x, y) = the two columns
#pragma unroll
  for (int i = 0; i < NI; ++i) {
    const float4 c0 = holds ? *reinterpret_cast<const float4*>(S_g + 64 * i + 4 * sub) : make_float4(0.f, 0.f, 0.f, 0.f);
    const float4 c1 = holds ? *reinterpret_cast<const float4*>(S_g + D + 64 * i + 4 * sub) : make_float4(0.f, 0.f, 0.f, 0.f);
    S_r[i][0] = make_float2(c0.x, c1.x);
    S_r[i][1] = make_float2(c0.y, c1.y);
    S_r[i][2] = make_float2(c0.z, c1.z);
    S_r[i][3] = make_float2(c0.w, c1.w);
  }
  const int Nc = m.n_conv();
  // ring entry: [k (D) | q (D) | v of the slice (CB) | beta, g, 0, 0]; all parts are whole 16-byte pieces
  const int n16 = (2 * D + CB) / 4, pitch = 2 * D + CB + 4;
  const float* k_src = prep + (size_t)m.Hk * D + (size_t)kh * D;
  const float* q_src = prep + (size_t)kh * D;
  const float* v_src = prep + (size_t)m.n_qk() + (size_t)h * Dv + blockIdx.z * CB;
  auto issue = [&](int i) {
    float* dst = sm + (size_t)(i % DELTA_RING) * pitch;
    const size_t row = (size_t)(r0 + i) * ldp;
    for (int e = threadIdx.x; e < n16 + 2; e += blockDim.x) {
      if (e < D / 4) cp_async16_ca(dst + 4 * e, k_src + row + 4 * e);
      else if (e < D / 2) cp_async16_ca(dst + 4 * e, q_src + row + 4 * (e - D / 4));
      else if (e < n16) cp_async16_ca(dst + 4 * e, v_src + row + 4 * (e - D / 2));
      else cp_async4(dst + 4 * n16 + (e - n16), prep + row + (e == n16 ? Nc + h : Nc + m.H + h));
    }
  };
#pragma unroll
  for (int s = 0; s < DELTA_RING - 1; ++s) {
    if (s < n) issue(s);
    asm volatile("cp.async.commit_group;" ::: "memory");
  }
  for (int i = 0; i < n; ++i) {
    asm volatile("cp.async.wait_group %0;" ::"n"(DELTA_RING - 2) : "memory");
    __syncthreads();                                         // token i's entry is there; token i-1's entry is read out
    if (i + DELTA_RING - 1 < n) issue(i + DELTA_RING - 1);
    asm volatile("cp.async.commit_group;" ::: "memory");
    const float* in = sm + (size_t)(i % DELTA_RING) * pitch;
    float4 kk[NI], qq[NI];
#pragma unroll
    for (int c = 0; c < NI; ++c) {
      kk[c] = holds ? *reinterpret_cast<const float4*>(in + 64 * c + 4 * sub) : make_float4(0.f, 0.f, 0.f, 0.f);
      qq[c] = holds ? *reinterpret_cast<const float4*>(in + D + 64 * c + 4 * sub) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    const float2 v = *reinterpret_cast<const float2*>(in + 2 * D + 2 * cg);
    const float beta = in[2 * D + CB], g = in[2 * D + CB + 1];
    float2 sk = make_float2(0.f, 0.f), sk2 = make_float2(0.f, 0.f);
#pragma unroll
    for (int c = 0; c < NI; ++c) {
      sk.x = fmaf(S_r[c][0].x, kk[c].x, sk.x);
      sk.y = fmaf(S_r[c][0].y, kk[c].x, sk.y);
      sk2.x = fmaf(S_r[c][1].x, kk[c].y, sk2.x);
      sk2.y = fmaf(S_r[c][1].y, kk[c].y, sk2.y);
      sk.x = fmaf(S_r[c][2].x, kk[c].z, sk.x);
      sk.y = fmaf(S_r[c][2].y, kk[c].z, sk.y);
      sk2.x = fmaf(S_r[c][3].x, kk[c].w, sk2.x);
      sk2.y = fmaf(S_r[c][3].y, kk[c].w, sk2.y);
    }
    sk.x += sk2.x;
    sk.y += sk2.y;
#pragma unroll
    for (int o = 1; o < 16; o <<= 1) {
      sk.x += __shfl_xor_sync(0xffffffffu, sk.x, o);
      sk.y += __shfl_xor_sync(0xffffffffu, sk.y, o);
    }
    const float ux = beta * (v.x - g * sk.x), uy = beta * (v.y - g * sk.y);
    float2 o2 = make_float2(0.f, 0.f), o3 = make_float2(0.f, 0.f);
#pragma unroll
    for (int c = 0; c < NI; ++c) {
      const float ke[4] = {kk[c].x, kk[c].y, kk[c].z, kk[c].w};
      const float qe[4] = {qq[c].x, qq[c].y, qq[c].z, qq[c].w};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        float2 s = S_r[c][e];
        s.x = fmaf(ke[e], ux, g * s.x);
        s.y = fmaf(ke[e], uy, g * s.y);
        S_r[c][e] = s;
        if (e & 1) {
          o3.x = fmaf(s.x, qe[e], o3.x);
          o3.y = fmaf(s.y, qe[e], o3.y);
        } else {
          o2.x = fmaf(s.x, qe[e], o2.x);
          o2.y = fmaf(s.y, qe[e], o2.y);
        }
      }
    }
    o2.x += o3.x;
    o2.y += o3.y;
#pragma unroll
    for (int o = 1; o < 16; o <<= 1) {
      o2.x += __shfl_xor_sync(0xffffffffu, o2.x, o);
      o2.y += __shfl_xor_sync(0xffffffffu, o2.y, o);
    }
    if (sub == 0) *reinterpret_cast<float2*>(o_raw + (size_t)(r0 + i) * ldo + (size_t)h * Dv + col0) = o2;
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");
  if (write_state && holds) {
#pragma unroll
    for (int i = 0; i < NI; ++i) {
      *reinterpret_cast<float4*>(S_g + 64 * i + 4 * sub) = make_float4(S_r[i][0].x, S_r[i][1].x, S_r[i][2].x, S_r[i][3].x);
      *reinterpret_cast<float4*>(S_g + D + 64 * i + 4 * sub) = make_float4(S_r[i][0].y, S_r[i][1].y, S_r[i][2].y, S_r[i][3].y);
    }
  }
}

template <int D>
int launch_delta_recurrence_quad(const float* prep, long ldp, DeltaDims m, float* state, const int32_t* seq_q_start,
                                 const int32_t* seq_slot, float* o_raw, long ldo, int n_seqs, int write_state,
                                 cudaStream_t stream) {
  const int CB = m.Dv % 32 == 0 ? 32 : 16;                   // columns per block
  const size_t smem = (size_t)DELTA_RING * (2 * D + CB + 4) * sizeof(float);
  return launch_pdl(PDL_ATTENTION, delta_recurrence_quad_kernel<D>, dim3(m.H, n_seqs, m.Dv / CB), dim3(8 * CB), smem, stream, prep,
                    ldp, m, state, seq_q_start, seq_slot, o_raw, ldo, write_state);
}

// One warp per (token, head): out = o / sqrt(mean(o^2) + eps) * w * act(gate); w is one vector for all heads
// (w_head_stride 0) or a vector per head (w_head_stride Dv); act: silu (0) or the logistic function (1).
template <typename T>
__global__ void __launch_bounds__(128)
delta_finish_kernel(const float* __restrict__ o_raw, long ldo, const float* __restrict__ gate, long ldg,
                    const float* __restrict__ w_all, int w_head_stride, int gate_act, float eps, int H, int Dv,
                    const int32_t* __restrict__ tok_seq, T* __restrict__ out, long ld_out, long n_items) {
  pdl_launch_dependents();
  pdl_wait();
  const long item = (long)blockIdx.x * 4 + (threadIdx.x >> 5);
  if (item >= n_items) return;
  const int lane = threadIdx.x & 31;
  const int t = (int)(item / H), h = (int)(item - (long)t * H);
  T* dst = out + (size_t)t * ld_out + (size_t)h * Dv;
  if (tok_seq[t] < 0) {
    for (int d = lane; d < Dv; d += 32) dst[d] = from_f32<T>(0.f);
    return;
  }
  const float* o = o_raw + (size_t)t * ldo + (size_t)h * Dv;
  const float* g = gate + (size_t)t * ldg + (size_t)h * Dv;
  const float* w = w_all + (size_t)h * w_head_stride;
  float ss = 0.f;
  for (int d = lane; d < Dv; d += 32) ss = fmaf(o[d], o[d], ss);
  ss = warp_sum(ss);
  const float sc = 1.0f / sqrtf(ss / (float)Dv + eps);
  for (int d = lane; d < Dv; d += 32)
    dst[d] = from_f32<T>(w[d] * (o[d] * sc) * (gate_act == 0 ? silu_f(g[d]) : 1.0f / (1.0f + expf(-g[d]))));
}

// The same for ONE wide "head" per token (a norm over a whole row of many entries): a block per token.
template <typename T>
__global__ void __launch_bounds__(256)
delta_finish_row_kernel(const float* __restrict__ o_raw, long ldo, const float* __restrict__ gate, long ldg,
                        const float* __restrict__ w, int gate_act, float eps, int Dv, const int32_t* __restrict__ tok_seq,
                        T* __restrict__ out, long ld_out) {
  __shared__ float scratch[32];
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  T* dst = out + (size_t)t * ld_out;
  if (tok_seq[t] < 0) {
    for (int d = threadIdx.x; d < Dv; d += blockDim.x) dst[d] = from_f32<T>(0.f);
    return;
  }
  const float* o = o_raw + (size_t)t * ldo;
  const float* g = gate + (size_t)t * ldg;
  float ss = 0.f;
  for (int d = threadIdx.x; d < Dv; d += blockDim.x) ss = fmaf(o[d], o[d], ss);
  ss = block_sum(ss, scratch);
  const float sc = 1.0f / sqrtf(ss / (float)Dv + eps);
  for (int d = threadIdx.x; d < Dv; d += blockDim.x)
    dst[d] = from_f32<T>(w[d] * (o[d] * sc) * (gate_act == 0 ? silu_f(g[d]) : 1.0f / (1.0f + expf(-g[d]))));
}

template <int DREG>
int launch_delta_recurrence(const float* prep, long ldp, DeltaDims m, float* state, const int32_t* seq_q_start,
                            const int32_t* seq_slot, float* o_raw, long ldo, int n_seqs, int write_state,
                            cudaStream_t stream) {
  const int cols = (m.Dv + 31) / 32 * 32;
  const size_t smem = ((size_t)4 * m.D + (DREG > 0 ? 0 : (size_t)m.D * cols)) * sizeof(float);
  static PerDevice<size_t> allowed;
  if (smem > 48 * 1024 && allowed.here() < smem) {
    if (cudaFuncSetAttribute(delta_recurrence_kernel<DREG>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
      return LLMI_ERR_BAD_SIZE;
    allowed.here() = smem;
  }
  return launch_pdl(PDL_ATTENTION, delta_recurrence_kernel<DREG>, dim3(m.H, n_seqs), dim3(cols), smem, stream, prep, ldp, m, state,
                    seq_q_start, seq_slot, o_raw, ldo, write_state);
}

}  // namespace llmi

using namespace llmi;

static int delta_dims_ok(const DeltaDims& m) {
  return m.H > 0 && m.Hk > 0 && m.D > 0 && m.Dv > 0 && m.taps >= 1 && m.taps <= DELTA_MAX_TAPS && m.H % m.Hk == 0 && m.Dv <= 1024;
}

LLMI_EXPORT long llmi_delta_state_floats(int H, int Hk, int D, int Dv, int taps) {
  return DeltaDims{H, Hk, D, Dv, taps}.state_floats();
}

LLMI_EXPORT int llmi_delta_prepare(const float* proj, long ld, int H, int Hk, int D, int Dv, int taps, const float* conv_w,
                                   const float* a_log, const float* dt_bias, const float* state, const int32_t* tok_seq,
                                   const int32_t* tok_pos, const int32_t* seq_q_start, const int32_t* seq_slot, float* prep,
                                   long ldp, int n_tokens, cudaStream_t stream) {
  const DeltaDims m{H, Hk, D, Dv, taps};
  if (n_tokens <= 0 || !delta_dims_ok(m)) return LLMI_ERR_BAD_SIZE;
  const int pieces = 2 * m.Hk + (m.H * m.Dv + DELTA_V_PIECE - 1) / DELTA_V_PIECE;
  if (pieces > 65535) return LLMI_ERR_BAD_SIZE;
  const int threads = m.D >= 256 ? 256 : (m.D > 64 ? 128 : 64);
  return launch_pdl(PDL_SMALL, delta_prepare_kernel, dim3(n_tokens, pieces), dim3(threads), 0, stream, proj, ld, m, conv_w, a_log,
                    dt_bias, state, tok_seq, tok_pos, seq_q_start, seq_slot, prep, ldp);
}

LLMI_EXPORT int llmi_delta_conv_carry(const float* proj, long ld, int H, int Hk, int D, int Dv, int taps, float* state,
                                      const int32_t* seq_q_start, const int32_t* seq_kv_len, const int32_t* seq_slot,
                                      int n_seqs, cudaStream_t stream) {
  const DeltaDims m{H, Hk, D, Dv, taps};
  if (n_seqs <= 0 || n_seqs > 65535 || !delta_dims_ok(m)) return LLMI_ERR_BAD_SIZE;
  if (taps <= 1) return LLMI_OK;
  return launch_pdl(PDL_SMALL, delta_conv_carry_kernel, dim3((m.n_conv() + 127) / 128, n_seqs), dim3(128), 0, stream, proj, ld, m,
                    state, seq_q_start, seq_kv_len, seq_slot, n_seqs);
}

LLMI_EXPORT int llmi_delta_recurrence(const float* prep, long ldp, int H, int Hk, int D, int Dv, int taps, float* state,
                                      const int32_t* seq_q_start, const int32_t* seq_slot, float* o_raw, long ldo, int n_seqs,
                                      int write_state, cudaStream_t stream) {
  const DeltaDims m{H, Hk, D, Dv, taps};
  if (n_seqs <= 0 || n_seqs > 65535 || !delta_dims_ok(m)) return LLMI_ERR_BAD_SIZE;
  // (16-byte accesses: state rows, o rows and the ring's v entries must be 16-byte aligned)
  if (Dv % 16 == 0 && ldo % 4 == 0 && ldp % 4 == 0 && !((uintptr_t)state & 15) && !((uintptr_t)o_raw & 15) &&
      !((uintptr_t)prep & 15) && DeltaDims{H, Hk, D, Dv, taps}.state_floats() % 4 == 0) {
    if (D == 32) return launch_delta_recurrence_quad<32>(prep, ldp, m, state, seq_q_start, seq_slot, o_raw, ldo, n_seqs, write_state, stream);
    if (D == 64) return launch_delta_recurrence_quad<64>(prep, ldp, m, state, seq_q_start, seq_slot, o_raw, ldo, n_seqs, write_state, stream);
    if (D == 128) return launch_delta_recurrence_quad<128>(prep, ldp, m, state, seq_q_start, seq_slot, o_raw, ldo, n_seqs, write_state, stream);
  }
  if ((size_t)D * ((Dv + 31) / 32 * 32) * 4 + 16 * (size_t)D > 200 * 1024) return LLMI_ERR_BAD_SIZE;
  return launch_delta_recurrence<0>(prep, ldp, m, state, seq_q_start, seq_slot, o_raw, ldo, n_seqs, write_state, stream);
}

LLMI_EXPORT int llmi_delta_finish(int dtype, const float* o_raw, long ldo, const float* gate, long ldg, const float* w,
                                  int w_head_stride, int gate_act, float eps, int H, int Dv, const int32_t* tok_seq, void* out,
                                  long ld_out, int n_tokens, cudaStream_t stream) {
  if (n_tokens <= 0 || H <= 0 || Dv <= 0 || (w_head_stride != 0 && w_head_stride != Dv)) return LLMI_ERR_BAD_SIZE;
  if (gate_act != 0 && gate_act != 1) return LLMI_ERR_UNSUPPORTED;
  const long items = (long)n_tokens * H;
  const unsigned blocks = (unsigned)((items + 3) / 4);
  if (H == 1 && Dv >= 512) {
    if (dtype == LLMI_DTYPE_F32)
      return launch_pdl(PDL_SMALL, delta_finish_row_kernel<float>, dim3(n_tokens), dim3(256), 0, stream, o_raw, ldo, gate, ldg, w,
                        gate_act, eps, Dv, tok_seq, (float*)out, ld_out);
    if (dtype == LLMI_DTYPE_BF16)
      return launch_pdl(PDL_SMALL, delta_finish_row_kernel<__nv_bfloat16>, dim3(n_tokens), dim3(256), 0, stream, o_raw, ldo, gate,
                        ldg, w, gate_act, eps, Dv, tok_seq, (__nv_bfloat16*)out, ld_out);
    return LLMI_ERR_BAD_DTYPE;
  }
  if (dtype == LLMI_DTYPE_F32)
    return launch_pdl(PDL_SMALL, delta_finish_kernel<float>, blocks, 128, 0, stream, o_raw, ldo, gate, ldg, w, w_head_stride,
                      gate_act, eps, H, Dv, tok_seq, (float*)out, ld_out, items);
  if (dtype == LLMI_DTYPE_BF16)
    return launch_pdl(PDL_SMALL, delta_finish_kernel<__nv_bfloat16>, blocks, 128, 0, stream, o_raw, ldo, gate, ldg, w,
                      w_head_stride, gate_act, eps, H, Dv, tok_seq, (__nv_bfloat16*)out, ld_out, items);
  return LLMI_ERR_BAD_DTYPE;
}
