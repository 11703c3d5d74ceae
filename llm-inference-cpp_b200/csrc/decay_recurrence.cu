// Linear attention with a decay: a recurrent mixer whose per-head state S [D, Dv] forgets by a factor per token and
// takes one outer product:
//     S <- diag(w) S + k vᵀ ;        o = q_scale * Sᵀ q
// w is either a vector over the D key channels made anew for every token (a gate per channel: `dec` rows), or ONE
// constant number per head (`head_decay`).  Column j of S evolves alone:  s_j <- w * s_j + k v_j,  o_j = s_j . q — so
// the state is kept column by column ([head][column][entry], fp32, one row of the cache's state slab per slot) and the
// columns are spread over threads.  There is no sum over the state on the chain from token to token (unlike the delta
// rules of delta_rule.cu and dplr_delta.cu): a token is D/16 fused multiply-adds a thread.
//
// Everything here is fp32 arithmetic.  Kernels, in the order of a step:
//   llmi_channel_decay      per (token, head): w = logistic(z)^(1/tau), z = bias + W2 low (a low-rank path's second
//                           product, walked here), as exp(log_logistic(z) / tau)
//   llmi_rows_activate      an activation on the first columns of fp32 rows, in place (q, k, v through silu)
//   llmi_decay_recurrence   per (sequence, head, slice of columns): the recurrence over the step's tokens
//   (llmi_delta_finish of delta_rule.cu then norms and gates o)
// The recurrence treats a column alone and only continues what the slab holds: the result does not depend on how a
// prompt was cut or on what else is in the batch.
#include <math.h>

#include "common.cuh"

namespace llmi {

// log(logistic(z)) without overflow: -softplus(-z).
__device__ __forceinline__ float log_logistic(float z) { return z < 0.f ? z - log1pf(expf(z)) : -log1pf(expf(-z)); }

// `low` fp32 rows [T, ld] (R entries from column 0 of the pointer); w2t fp32 [R, H*D] (the second matrix transposed:
// neighbouring threads read neighbours); bias fp32 [H*D]; dec fp32 [T, ldd] receives the decays.  A block takes
// DECAY_PREP_TOK tokens and blockDim.x channels: an entry of w2t is read once for all of the block's tokens; a token's
// sum runs over j in ascending order whatever tokens share its block.
constexpr int DECAY_PREP_TOK = 8;
template <int TOKS>
__global__ void __launch_bounds__(256)
channel_decay_kernel(const float* __restrict__ low, long ld, int R, const float* __restrict__ w2t, const float* __restrict__ bias,
                     float inv_tau, int N, int n_tokens, const int32_t* __restrict__ tok_seq, float* __restrict__ dec, long ldd) {
  extern __shared__ float low_s[];                           // [TOKS][R]
  pdl_launch_dependents();
  pdl_wait();
  const int t0 = blockIdx.x * TOKS, cnt = min(TOKS, n_tokens - t0);
  for (int x = threadIdx.x; x < cnt * R; x += blockDim.x) {
    const int tt = x / R, j = x - tt * R;
    low_s[x] = low[(size_t)(t0 + tt) * ld + j];
  }
  __syncthreads();
  const int c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= N) return;
  float z[TOKS];
  const float b = bias ? bias[c] : 0.f;
#pragma unroll
  for (int tt = 0; tt < TOKS; ++tt) z[tt] = b;
#pragma unroll 8
  for (int j = 0; j < R; ++j) {
    const float w = w2t[(size_t)j * N + c];
#pragma unroll
    for (int tt = 0; tt < TOKS; ++tt)
      if (tt < cnt) z[tt] = fmaf(w, low_s[tt * R + j], z[tt]);
  }
#pragma unroll
  for (int tt = 0; tt < TOKS; ++tt)
    if (tt < cnt && tok_seq[t0 + tt] >= 0) dec[(size_t)(t0 + tt) * ldd + c] = expf(log_logistic(z[tt]) * inv_tau);
}

// The same for a handful of tokens, from the second matrix as stored (w2 fp32 [N, R], a channel's R entries side by
// side): a thread owns one channel of one token and reads its row in 16-byte pieces, all of them under way at once; the
// sum runs over j in ascending order, as above.
__global__ void __launch_bounds__(64)
channel_decay_rows_kernel(const float* __restrict__ low, long ld, int R, const float* __restrict__ w2, const float* __restrict__ bias,
                          float inv_tau, int N, const int32_t* __restrict__ tok_seq, float* __restrict__ dec, long ldd) {
  extern __shared__ __align__(16) float low_s[];
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  if (tok_seq[t] < 0) return;
  for (int j = threadIdx.x; j < R; j += blockDim.x) low_s[j] = low[(size_t)t * ld + j];
  __syncthreads();
  const int c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= N) return;
  float z = bias ? bias[c] : 0.f;
  const float4* row = reinterpret_cast<const float4*>(w2 + (size_t)c * R);
#pragma unroll 4
  for (int j4 = 0; j4 < R / 4; ++j4) {
    const float4 w = row[j4];
    const float4 l = *reinterpret_cast<const float4*>(low_s + 4 * j4);
    z = fmaf(w.x, l.x, z);
    z = fmaf(w.y, l.y, z);
    z = fmaf(w.z, l.z, z);
    z = fmaf(w.w, l.w, z);
  }
  dec[(size_t)t * ldd + c] = expf(log_logistic(z) * inv_tau);
}

// x[t, 0:n] = act(x[t, 0:n]) in place; act 0: silu.
__global__ void __launch_bounds__(256)
rows_activate_kernel(float* __restrict__ x, long ld, int n, long total, int act) {
  pdl_launch_dependents();
  pdl_wait();
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long)gridDim.x * blockDim.x) {
    const long t = i / n;
    float* p = x + t * ld + (i - t * n);
    const float v = *p;
    *p = v / (1.0f + expf(-v));
  }
}

// The same for rows of whole 16-byte pieces: n4 = n / 4 pieces a row.
__global__ void __launch_bounds__(256)
rows_activate_vec4_kernel(float* __restrict__ x, long ld, int n4, long total4, int act) {
  pdl_launch_dependents();
  pdl_wait();
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < total4; i += (long)gridDim.x * blockDim.x) {
    const long t = i / n4;
    float4* p = reinterpret_cast<float4*>(x + t * ld) + (i - t * n4);
    float4 v = *p;
    v.x = v.x / (1.0f + expf(-v.x));
    v.y = v.y / (1.0f + expf(-v.y));
    v.z = v.z / (1.0f + expf(-v.z));
    v.w = v.w / (1.0f + expf(-v.w));
    *p = v;
  }
}

// Where a token's vectors lie: q, k, v in the fp32 rows `proj` (column offsets; heads side by side), the decays of the
// key channels in `dec` rows, or one number per head.
struct DecaySources {
  const float* proj;
  long ld;
  int q_off, k_off, v_off;
  const float* dec;          // [T, ldw] or null
  long ldw;
  const float* head_decay;   // [H] or null
  float q_scale;
  int silu_in;               // q, k, v pass silu as they are read (a step of a handful of tokens: no pass of its own over the rows)
};

__device__ __forceinline__ float decay_silu(float v) { return v / (1.0f + expf(-v)); }

// The general form: one block per (head, sequence), one thread per column j of S, the column in shared memory
// (S_s[d][cols]: no two threads share a bank); any D and Dv.  The vectors of the next token are fetched while the
// current one is computed (two buffers, one barrier per token).
__global__ void __launch_bounds__(1024)
decay_recurrence_kernel(DecaySources a, int H, int D, int Dv, float* __restrict__ state, long state_stride,
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
  const int cols = blockDim.x;                               // Dv rounded up to whole warps
  const int j = threadIdx.x;
  const bool live = j < Dv;
  float* vec = sm;                                           // [2][3*D]: w, k, q of a token
  float* S_s = sm + 6 * D;                                   // [D][cols]
  float* S_g = state + (size_t)slot * state_stride + (size_t)h * D * Dv;
  if (live)
    for (int d = 0; d < D; ++d) S_s[(size_t)d * cols + j] = S_g[(size_t)j * D + d];
  const float wh = a.head_decay ? a.head_decay[h] : 0.f;
  auto fetch = [&](int i, int buf) {
    const float* xr = a.proj + (size_t)(r0 + i) * a.ld + (size_t)h * D;
    float* dst = vec + buf * 3 * D;
    for (int d = threadIdx.x; d < D; d += blockDim.x) {
      dst[d] = a.dec ? a.dec[(size_t)(r0 + i) * a.ldw + (size_t)h * D + d] : wh;
      dst[D + d] = a.silu_in ? decay_silu(xr[a.k_off + d]) : xr[a.k_off + d];
      dst[2 * D + d] = a.silu_in ? decay_silu(xr[a.q_off + d]) : xr[a.q_off + d];
    }
  };
  fetch(0, 0);
  for (int i = 0; i < n; ++i) {
    __syncthreads();                                         // buffer i&1 is filled; the other one is read out
    if (i + 1 < n) fetch(i + 1, (i + 1) & 1);
    if (!live) continue;
    float v = a.proj[(size_t)(r0 + i) * a.ld + a.v_off + (size_t)h * Dv + j];
    if (a.silu_in) v = decay_silu(v);
    const float* w = vec + (i & 1) * 3 * D;
    const float *k = w + D, *q = w + 2 * D;
    float o = 0.f;
    for (int d = 0; d < D; ++d) {
      const float s = fmaf(k[d], v, w[d] * S_s[(size_t)d * cols + j]);
      S_s[(size_t)d * cols + j] = s;
      o = fmaf(s, q[d], o);
    }
    o_raw[(size_t)(r0 + i) * ldo + (size_t)h * Dv + j] = o * a.q_scale;
  }
  if (live && write_state)
    for (int d = 0; d < D; ++d) S_g[(size_t)j * D + d] = S_s[(size_t)d * cols + j];
}

// The form for D a multiple of 4 up to 256 and Dv a multiple of 16.  A thread holds TWO neighbouring columns of S and
// a sixteenth of their entries (lane `sub` of sixteen: d = 64 i + 4 sub + 0..3, while d < D) in registers; the partial
// sums of o over d of a stage's eight tokens (sixteen numbers a thread) are joined over the sixteen lanes at the stage's
// end by a butterfly that halves what a lane keeps in every round (fifteen shuffles for eight tokens; lane i ends up
// with number i: token i / 2, column i % 2), off the chain from token to token.  A head's columns
// are cut into slices of 32 (or 16), every slice a block of its own (blockIdx.z).  What the tokens need — w (unless the
// decay is a number per head), k, q of the head, the slice's v — is copied into a ring of DECAY_RING stages of
// DECAY_TOK tokens each, DECAY_RING - 1 stages ahead (cp.async, 16 bytes a copy), so that no load's latency lies on the
// chain; ONE barrier per stage: nothing on the chain from token to token needs another thread (a token is two dependent
// operations per state entry), so a barrier per token would be most of a token's time.
constexpr int DECAY_RING = 4, DECAY_TOK = 8;      // (eight tokens x two columns = the sixteen lanes of the butterfly)

__device__ __forceinline__ void decay_cp16(void* dst, const void* src) {
  const uint32_t d = (uint32_t)__cvta_generic_to_shared(dst);
  asm volatile("cp.async.ca.shared.global [%0], [%1], 16;" ::"r"(d), "l"(src) : "memory");
}

template <int NI, bool SCALAR, bool SILU>
__global__ void __launch_bounds__(256)
decay_recurrence_lanes_kernel(DecaySources a, int H, int D, int Dv, float* __restrict__ state, long state_stride,
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
  const int CB = blockDim.x >> 3;                            // columns of this block's slice (the launcher gives 8 CB threads)
  const int cg = threadIdx.x >> 4, sub = threadIdx.x & 15;   // my columns: col0, col0 + 1
  const int col0 = blockIdx.z * CB + 2 * cg;
  bool holds[NI];
#pragma unroll
  for (int i = 0; i < NI; ++i) holds[i] = 64 * i + 4 * sub < D;
  float* S_g = state + (size_t)slot * state_stride + (size_t)h * D * Dv + (size_t)col0 * D;     // [column][entry]
  float2 S_r[NI][4];                                         // [chunk][entry of the chunk] . (x, y) = the two columns
  const float4 zero = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
  for (int i = 0; i < NI; ++i) {
    const float4 c0 = holds[i] ? *reinterpret_cast<const float4*>(S_g + 64 * i + 4 * sub) : zero;
    const float4 c1 = holds[i] ? *reinterpret_cast<const float4*>(S_g + D + 64 * i + 4 * sub) : zero;
    S_r[i][0] = make_float2(c0.x, c1.x);
    S_r[i][1] = make_float2(c0.y, c1.y);
    S_r[i][2] = make_float2(c0.z, c1.z);
    S_r[i][3] = make_float2(c0.w, c1.w);
  }
  // a token's entry of a stage: [w (D, unless SCALAR) | k (D) | q (D) | v of the slice (CB)]; all parts are whole 16-byte pieces
  constexpr int NVEC = SCALAR ? 2 : 3;
  const int Q = D / 4;                                       // 16-byte pieces of one vector
  const int n16 = NVEC * Q + CB / 4, pitch = NVEC * D + CB;
  const float* v_src = a.proj + a.v_off + (size_t)h * Dv + blockIdx.z * CB;
  const float* k_src = a.proj + a.k_off + (size_t)h * D;
  const float* q_src = a.proj + a.q_off + (size_t)h * D;
  const float* w_src = SCALAR ? nullptr : a.dec + (size_t)h * D;
  const int n_stages = (n + DECAY_TOK - 1) / DECAY_TOK;
  // a token's entry has at most 3 * 32 + 8 pieces (NI <= 2), fewer than the block has threads, or 3 * 64 + 8 (NI = 4), no
  // more than twice as many: thread e copies piece e (and e + blockDim.x) of every token, from an address that moves by
  // one row a token
  constexpr int SLOTS = NI > 2 ? 2 : 1;
  const float* my_src[SLOTS];
  long my_step[SLOTS];
#pragma unroll
  for (int u = 0; u < SLOTS; ++u) {
    my_src[u] = nullptr;
    my_step[u] = 0;
    const int e = threadIdx.x + u * blockDim.x;
    if (e >= n16) continue;
    const int part = e / Q, off = 4 * (e - part * Q);
    const int which = SCALAR ? part + 1 : part;              // 0: w, 1: k, 2: q, 3: v
    my_step[u] = which == 0 ? a.ldw : a.ld;
    my_src[u] = (which == 0 ? w_src + off : which == 1 ? k_src + off : which == 2 ? q_src + off : v_src + 4 * (e - NVEC * Q)) +
                (size_t)r0 * my_step[u];
  }
  auto issue = [&](int st) {
    const int t0 = st * DECAY_TOK, cnt = min(DECAY_TOK, n - t0);
#pragma unroll
    for (int u = 0; u < SLOTS; ++u) {
      if (!my_src[u]) continue;
      float* dst = sm + (size_t)(st % DECAY_RING) * DECAY_TOK * pitch + 4 * (threadIdx.x + u * blockDim.x);
      const float* src = my_src[u] + (size_t)t0 * my_step[u];
#pragma unroll
      for (int tk = 0; tk < DECAY_TOK; ++tk)
        if (tk < cnt) decay_cp16(dst + (size_t)tk * pitch, src + (size_t)tk * my_step[u]);
    }
  };
#pragma unroll
  for (int s = 0; s < DECAY_RING - 1; ++s) {
    if (s < n_stages) issue(s);
    asm volatile("cp.async.commit_group;" ::: "memory");
  }
  const float wh = SCALAR ? a.head_decay[h] : 0.f;
  float* o_dst = o_raw + (size_t)r0 * ldo + (size_t)h * Dv + col0;
  for (int st = 0; st < n_stages; ++st) {
    asm volatile("cp.async.wait_group %0;" ::"n"(DECAY_RING - 2) : "memory");
    __syncthreads();                                         // stage st is there; stage st-1 is read out
    if (st + DECAY_RING - 1 < n_stages) issue(st + DECAY_RING - 1);
    asm volatile("cp.async.commit_group;" ::: "memory");
    const float* stage = sm + (size_t)(st % DECAY_RING) * DECAY_TOK * pitch;
    const int t0 = st * DECAY_TOK, cnt = min(DECAY_TOK, n - t0);
    float part[2 * DECAY_TOK];                               // my part of S . q: [token][column]
    auto token = [&](const float* in, float& p0, float& p1) {
      float2 v = *reinterpret_cast<const float2*>(in + NVEC * D + 2 * cg);
      if (SILU) v = make_float2(decay_silu(v.x), decay_silu(v.y));
      float2 o2 = make_float2(0.f, 0.f), o3 = make_float2(0.f, 0.f);
#pragma unroll
      for (int c = 0; c < NI; ++c) {
        const float4 ww = SCALAR ? make_float4(wh, wh, wh, wh) : (holds[c] ? *reinterpret_cast<const float4*>(in + 64 * c + 4 * sub) : zero);
        const float4 kk = holds[c] ? *reinterpret_cast<const float4*>(in + (NVEC - 2) * D + 64 * c + 4 * sub) : zero;
        const float4 qq = holds[c] ? *reinterpret_cast<const float4*>(in + (NVEC - 1) * D + 64 * c + 4 * sub) : zero;
        const float we[4] = {ww.x, ww.y, ww.z, ww.w};
        float ke[4] = {kk.x, kk.y, kk.z, kk.w}, qe[4] = {qq.x, qq.y, qq.z, qq.w};
        if (SILU) {
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            ke[e] = decay_silu(ke[e]);
            qe[e] = decay_silu(qe[e]);
          }
        }
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          float2 s = S_r[c][e];
          s.x = fmaf(ke[e], v.x, we[e] * s.x);
          s.y = fmaf(ke[e], v.y, we[e] * s.y);
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
      p0 = o2.x + o3.x;
      p1 = o2.y + o3.y;
    };
    if (cnt == DECAY_TOK) {                                  // a whole stage: nothing between its tokens but the chain itself
#pragma unroll
      for (int tk = 0; tk < DECAY_TOK; ++tk) token(stage + (size_t)tk * pitch, part[2 * tk], part[2 * tk + 1]);
    } else {
#pragma unroll
      for (int tk = 0; tk < DECAY_TOK; ++tk) {
        part[2 * tk] = 0.f;
        part[2 * tk + 1] = 0.f;
        if (tk < cnt) token(stage + (size_t)tk * pitch, part[2 * tk], part[2 * tk + 1]);
      }
    }
    // sixteen numbers a lane, sixteen lanes: every round a lane hands one half of what it holds to its partner and adds
    // the partner's other half to its own; lane `sub` is left with number `sub`.  Every number's sum has the same shape.
#pragma unroll
    for (int off = 8, half = DECAY_TOK; off >= 1; off >>= 1, half >>= 1) {
      const bool upper = (sub & off) != 0;
#pragma unroll
      for (int i = 0; i < half; ++i) {
        const float send = upper ? part[i] : part[i + half];
        const float keep = upper ? part[i + half] : part[i];
        part[i] = keep + __shfl_xor_sync(0xffffffffu, send, off);
      }
    }
    if ((sub >> 1) < cnt) o_dst[(size_t)(t0 + (sub >> 1)) * ldo + (sub & 1)] = part[0] * a.q_scale;
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");
  if (write_state) {
#pragma unroll
    for (int i = 0; i < NI; ++i) {
      if (!holds[i]) continue;
      *reinterpret_cast<float4*>(S_g + 64 * i + 4 * sub) = make_float4(S_r[i][0].x, S_r[i][1].x, S_r[i][2].x, S_r[i][3].x);
      *reinterpret_cast<float4*>(S_g + D + 64 * i + 4 * sub) = make_float4(S_r[i][0].y, S_r[i][1].y, S_r[i][2].y, S_r[i][3].y);
    }
  }
}

template <int NI, bool SCALAR, bool SILU>
int launch_decay_lanes(const DecaySources& a, int H, int D, int Dv, float* state, long state_stride, const int32_t* seq_q_start,
                       const int32_t* seq_slot, float* o_raw, long ldo, int n_seqs, int write_state, cudaStream_t stream) {
  // columns per block: 32, or 16 where that gives the device more blocks than it has SMs to fill (the chain over a
  // sequence's tokens is what a block's time is, however few columns it holds)
  const int CB = (Dv % 32 == 0 && (long)H * n_seqs * (Dv / 32) >= 2L * sm_count()) ? 32 : 16;
  const size_t smem = (size_t)DECAY_RING * DECAY_TOK * ((SCALAR ? 2 : 3) * D + CB) * sizeof(float);
  static PerDevice<size_t> allowed;
  if (smem > 48 * 1024 && allowed.here() < smem) {
    if (cudaFuncSetAttribute(decay_recurrence_lanes_kernel<NI, SCALAR, SILU>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
      return LLMI_ERR_BAD_SIZE;
    allowed.here() = smem;
  }
  return launch_pdl(PDL_ATTENTION, decay_recurrence_lanes_kernel<NI, SCALAR, SILU>, dim3(H, n_seqs, Dv / CB), dim3(8 * CB), smem, stream,
                    a, H, D, Dv, state, state_stride, seq_q_start, seq_slot, o_raw, ldo, write_state);
}

}  // namespace llmi

using namespace llmi;

// low: fp32 rows [T, ld] whose first R entries are the low-rank path's first product; w2t fp32 [R, N]; bias fp32 [N] or
// null; dec fp32 [T, ldd]: dec[t, c] = logistic(bias[c] + sum_j w2t[j, c] low[t, j])^(1/tau).  w2 (optional): the same
// matrix as stored, fp32 [N, R], for the form of a handful of tokens.
LLMI_EXPORT int llmi_channel_decay(const float* low, long ld, int R, const float* w2t, const float* w2, const float* bias, float tau,
                                   int N, const int32_t* tok_seq, float* dec, long ldd, int n_tokens, cudaStream_t stream) {
  if (n_tokens <= 0 || N <= 0 || R <= 0 || R > 4096 || !(tau > 0.f)) return LLMI_ERR_BAD_SIZE;
  if (n_tokens <= 64 && w2 && R % 4 == 0 && !((uintptr_t)w2 & 15)) {
    const int cuts = (N + 63) / 64;
    if (cuts > 65535) return LLMI_ERR_BAD_SIZE;
    return launch_pdl(PDL_SMALL, channel_decay_rows_kernel, dim3(n_tokens, cuts), dim3(64), (size_t)R * sizeof(float), stream, low, ld,
                      R, w2, bias, 1.0f / tau, N, tok_seq, dec, ldd);
  }
  if (n_tokens <= 64) {        // a handful of tokens: a block per token and 64 channels, so that the device has blocks enough
    const int threads = N >= 64 ? 64 : (N + 31) / 32 * 32;
    const int cuts = (N + threads - 1) / threads;
    if (cuts > 65535) return LLMI_ERR_BAD_SIZE;
    return launch_pdl(PDL_SMALL, channel_decay_kernel<1>, dim3(n_tokens, cuts), dim3(threads), (size_t)R * sizeof(float), stream,
                      low, ld, R, w2t, bias, 1.0f / tau, N, n_tokens, tok_seq, dec, ldd);
  }
  const int threads = N >= 256 ? 256 : (N + 31) / 32 * 32;
  const int cuts = (N + threads - 1) / threads;
  if (cuts > 65535) return LLMI_ERR_BAD_SIZE;
  const size_t smem = (size_t)DECAY_PREP_TOK * R * sizeof(float);
  static PerDevice<size_t> allowed;
  if (smem > 48 * 1024 && allowed.here() < smem) {
    if (cudaFuncSetAttribute(channel_decay_kernel<DECAY_PREP_TOK>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
      return LLMI_ERR_BAD_SIZE;
    allowed.here() = smem;
  }
  return launch_pdl(PDL_SMALL, channel_decay_kernel<DECAY_PREP_TOK>, dim3((n_tokens + DECAY_PREP_TOK - 1) / DECAY_PREP_TOK, cuts),
                    dim3(threads), smem, stream, low, ld, R, w2t, bias, 1.0f / tau, N, n_tokens, tok_seq, dec, ldd);
}

// x fp32 [T, ld]: x[:, 0:n] = act(x[:, 0:n]) in place; act 0: silu.
LLMI_EXPORT int llmi_rows_activate(float* x, long ld, int n, int n_rows, int act, cudaStream_t stream) {
  if (n_rows <= 0 || n <= 0 || ld < n) return LLMI_ERR_BAD_SIZE;
  if (act != 0) return LLMI_ERR_UNSUPPORTED;
  const long total = (long)n_rows * n;
  const long most = (long)sm_count() * 16;
  if (n % 4 == 0 && ld % 4 == 0 && !((uintptr_t)x & 15)) {
    const long want4 = (total / 4 + 255) / 256;
    return launch_pdl(PDL_SMALL, rows_activate_vec4_kernel, dim3((unsigned)(want4 < most ? want4 : most)), dim3(256), 0, stream, x,
                      ld, n / 4, total / 4, act);
  }
  const long want = (total + 255) / 256;
  return launch_pdl(PDL_SMALL, rows_activate_kernel, dim3((unsigned)(want < most ? want : most)), dim3(256), 0, stream, x, ld, n,
                    total, act);
}

// proj fp32 [T, ld]: q at column q_off, k at k_off (H*D each), v at v_off (H*Dv); the decay: dec fp32 [T, ldw] (H*D a
// row, a factor per key channel) or head_decay fp32 [H] (one factor per head) — exactly one of the two;
// state fp32 [slots, state_stride >= H*D*Dv]; o_raw fp32 [T, ldo] receives q_scale * Sᵀ q.  silu_in: q, k, v are read
// through silu (the same values as after llmi_rows_activate on the rows).
LLMI_EXPORT int llmi_decay_recurrence(const float* proj, long ld, int q_off, int k_off, int v_off, const float* dec, long ldw,
                                      const float* head_decay, float q_scale, int H, int D, int Dv, float* state,
                                      long state_stride, const int32_t* seq_q_start, const int32_t* seq_slot, float* o_raw,
                                      long ldo, int n_seqs, int write_state, int silu_in, cudaStream_t stream) {
  if (n_seqs <= 0 || n_seqs > 65535 || H <= 0 || H > 65535 || D <= 0 || Dv <= 0 || Dv > 1024) return LLMI_ERR_BAD_SIZE;
  if ((dec == nullptr) == (head_decay == nullptr)) return LLMI_ERR_UNSUPPORTED;
  const DecaySources a{proj, ld, q_off, k_off, v_off, dec, ldw, head_decay, q_scale, silu_in};
  const bool aligned = ld % 4 == 0 && q_off % 4 == 0 && k_off % 4 == 0 && v_off % 4 == 0 && ldo % 4 == 0 && state_stride % 4 == 0 &&
                       !((uintptr_t)state & 15) && !((uintptr_t)o_raw & 15) && !((uintptr_t)proj & 15) &&
                       (!dec || (ldw % 4 == 0 && !((uintptr_t)dec & 15)));
  if (aligned && D % 4 == 0 && D <= 256 && Dv % 16 == 0) {
#define LLMI_LANES(NI, SC, SI)                                                                                             \
  return launch_decay_lanes<NI, SC, SI>(a, H, D, Dv, state, state_stride, seq_q_start, seq_slot, o_raw, ldo, n_seqs, write_state, stream)
    if (D <= 64) {
      if (silu_in) { if (dec) LLMI_LANES(1, false, true); else LLMI_LANES(1, true, true); }
      if (dec) LLMI_LANES(1, false, false); else LLMI_LANES(1, true, false);
    }
    if (D <= 128) {
      if (silu_in) { if (dec) LLMI_LANES(2, false, true); else LLMI_LANES(2, true, true); }
      if (dec) LLMI_LANES(2, false, false); else LLMI_LANES(2, true, false);
    }
    if (silu_in) { if (dec) LLMI_LANES(4, false, true); else LLMI_LANES(4, true, true); }
    if (dec) LLMI_LANES(4, false, false); else LLMI_LANES(4, true, false);
#undef LLMI_LANES
  }
  const int cols = (Dv + 31) / 32 * 32;
  const size_t smem = ((size_t)6 * D + (size_t)D * cols) * sizeof(float);
  if (smem > 200 * 1024) return LLMI_ERR_BAD_SIZE;
  static PerDevice<size_t> allowed;
  if (smem > 48 * 1024 && allowed.here() < smem) {
    if (cudaFuncSetAttribute(decay_recurrence_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
      return LLMI_ERR_BAD_SIZE;
    allowed.here() = smem;
  }
  return launch_pdl(PDL_ATTENTION, decay_recurrence_kernel, dim3(H, n_seqs), dim3(cols), smem, stream, a, H, D, Dv, state,
                    state_stride, seq_q_start, seq_slot, o_raw, ldo, write_state);
}
