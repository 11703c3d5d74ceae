// From a token's projected row to what attention reads: one kernel between the q/k/v product and the attention kernel.
//
// `proj` is one fp32 row per token: [ q: n_q_heads * dk | k: n_k_heads * dk | v: n_v_heads * dv ]  (k and v are absent
// for a layer that reads another layer's keys and values).  Per token, in this order:
//   * optionally an RMS norm over the WHOLE q part (all heads at once) with a weight per entry, and the same over
//     the whole k part:  y = x / sqrt(mean(x^2) + eps) * w;
//   * optionally the rotation of the first rot_dims entries of every q and k head by the angle float(pos) * inv_freq[i]:
//     pairs (i, i + rot_dims/2) (`pairing` 0) or neighbours (2i, 2i + 1) (`pairing` 1), cos and sin both times
//     `amplitude` (1: a plain rotation);
//   * q goes to `q_out` in the compute type; k and v go to the cache pages of (sequence, position).
// Keys and values may differ in their number of heads and in their head size (two page layouts).  With `v_from_k`
// the row has no v part: the values are the key rows as projected (after the norm, before the rotation), head for head.
// All arithmetic is fp32; one block per token, or, where no norm ties a part's heads together, one per (token, head).
#include "common.cuh"
#include "step_meta.cuh"

namespace llmi {

// One part (q or k) of a row: scale, weight, rotation; element e of head hd goes to dst(head) + e.
struct NoCopy {
  __device__ __forceinline__ void* operator()(int) const { return nullptr; }
};

// `plain(head)`: where the head's entries go as they are before the rotation (the values of a layer whose values are
// its keys), or null.
template <typename T, typename Dst, typename Plain>
__device__ __forceinline__ void prepare_part(const float* __restrict__ src, int n_heads, int dk, float sc,
                                             const float* __restrict__ w, const float* __restrict__ inv_freq, int rot_dims,
                                             int pairing, float amplitude, int pos, Dst dst, Plain plain) {
  const int half = rot_dims / 2, n = n_heads * dk;
  for (int idx = threadIdx.x; idx < n; idx += blockDim.x) {
    const int hd = idx / dk, e = idx - hd * dk;
    T* o = dst(hd);
    T* pl = (T*)plain(hd);
    if (pl) pl[e] = from_f32<T>(w ? w[idx] * (src[idx] * sc) : src[idx] * sc);
    if (e < half) {
      float s, c;
      sincosf((float)pos * inv_freq[e], &s, &c);
      s *= amplitude;
      c *= amplitude;
      const int i0 = pairing ? idx + e : idx, i1 = pairing ? idx + e + 1 : idx + half;      // (idx + e = head start + 2e)
      const float a = w ? w[i0] * (src[i0] * sc) : src[i0] * sc;
      const float b = w ? w[i1] * (src[i1] * sc) : src[i1] * sc;
      o[pairing ? 2 * e : e] = from_f32<T>(rot_lo(a, b, c, s));
      o[pairing ? 2 * e + 1 : e + half] = from_f32<T>(rot_hi(a, b, c, s));
    } else if (e >= rot_dims) {
      o[e] = from_f32<T>(w ? w[idx] * (src[idx] * sc) : src[idx] * sc);
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(128)
qkv_prepare_kernel(const float* __restrict__ proj, long ld, int n_q_heads, int n_k_heads, int dk, int n_v_heads, int dv,
                   const float* __restrict__ q_norm_w, const float* __restrict__ k_norm_w, float eps,
                   const float* __restrict__ inv_freq, int rot_dims, int pairing, float amplitude, int v_from_k,
                   const int32_t* __restrict__ tok_seq,
                   const int32_t* __restrict__ tok_pos, PagedKV kp, PagedKV vp, T* __restrict__ k_cache,
                   T* __restrict__ v_cache, T* __restrict__ q_out, long ldq, int has_kv, int write_kv) {
  __shared__ float scratch[32];
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const int seq = tok_seq[t];
  const int Nq = n_q_heads * dk, Nk = n_k_heads * dk, Nv = n_v_heads * dv;
  T* qo = q_out + (size_t)t * ldq;
  if (seq < 0) {
    for (int i = threadIdx.x; i < Nq; i += blockDim.x) qo[i] = from_f32<T>(0.f);
    return;
  }
  const int pos = tok_pos[t];
  const float* row = proj + (size_t)t * ld;
  float sq = 1.f, sk = 1.f;
  if (q_norm_w) {
    float ss = 0.f;
    for (int i = threadIdx.x; i < Nq; i += blockDim.x) ss = fmaf(row[i], row[i], ss);
    sq = 1.0f / sqrtf(block_sum(ss, scratch) / (float)Nq + eps);
  }
  prepare_part<T>(row, n_q_heads, dk, sq, q_norm_w, inv_freq, rot_dims, pairing, amplitude, pos,
                  [&](int hd) { return qo + (size_t)hd * dk; }, NoCopy());
  if (!has_kv || !write_kv) return;
  const float* krow = row + Nq;
  if (k_norm_w) {
    float ss = 0.f;
    for (int i = threadIdx.x; i < Nk; i += blockDim.x) ss = fmaf(krow[i], krow[i], ss);
    sk = 1.0f / sqrtf(block_sum(ss, scratch) / (float)Nk + eps);
  }
  if (v_from_k) {
    prepare_part<T>(krow, n_k_heads, dk, sk, k_norm_w, inv_freq, rot_dims, pairing, amplitude, pos,
                    [&](int hd) { return k_cache + kv_row_offset(kp, seq, pos, hd); },
                    [&](int hd) { return (void*)(v_cache + kv_row_offset(vp, seq, pos, hd)); });
    return;
  }
  prepare_part<T>(krow, n_k_heads, dk, sk, k_norm_w, inv_freq, rot_dims, pairing, amplitude, pos,
                  [&](int hd) { return k_cache + kv_row_offset(kp, seq, pos, hd); }, NoCopy());
  const float* vrow = krow + Nk;
  for (int idx = threadIdx.x; idx < Nv; idx += blockDim.x) {
    const int hd = idx / dv, e = idx - hd * dv;
    v_cache[kv_row_offset(vp, seq, pos, hd) + e] = from_f32<T>(vrow[idx]);
  }
}

// Without the norms over the whole q and k parts a head needs nothing of its neighbours: one block per (token, head) —
// the q heads, then the k heads, then (unless the values are the keys) the v heads — with the same arithmetic per entry.
template <typename T>
__device__ __forceinline__ void prepare_head(const float* __restrict__ proj, long ld, int n_q_heads, int n_k_heads, int dk, int dv,
                                             const float* __restrict__ inv_freq, int rot_dims, int pairing, float amplitude,
                                             int v_from_k, int seq, const int32_t* __restrict__ tok_pos, const PagedKV& kp,
                                             const PagedKV& vp, T* __restrict__ k_cache, T* __restrict__ v_cache,
                                             T* __restrict__ q_out, long ldq, int t, int hd) {
  if (hd < n_q_heads) {
    T* qo = q_out + (size_t)t * ldq + (size_t)hd * dk;
    if (seq < 0) {
      for (int i = threadIdx.x; i < dk; i += blockDim.x) qo[i] = from_f32<T>(0.f);
      return;
    }
    prepare_part<T>(proj + (size_t)t * ld + (size_t)hd * dk, 1, dk, 1.f, nullptr, inv_freq, rot_dims, pairing, amplitude, tok_pos[t],
                    [&](int) { return qo; }, NoCopy());
    return;
  }
  if (seq < 0) return;
  const int pos = tok_pos[t];
  const float* krow = proj + (size_t)t * ld + (size_t)n_q_heads * dk;
  if (hd < n_q_heads + n_k_heads) {
    const int kh = hd - n_q_heads;
    T* ko = k_cache + kv_row_offset(kp, seq, pos, kh);
    if (v_from_k) {
      T* vo = v_cache + kv_row_offset(vp, seq, pos, kh);
      prepare_part<T>(krow + (size_t)kh * dk, 1, dk, 1.f, nullptr, inv_freq, rot_dims, pairing, amplitude, pos,
                      [&](int) { return ko; }, [&](int) { return (void*)vo; });
    } else {
      prepare_part<T>(krow + (size_t)kh * dk, 1, dk, 1.f, nullptr, inv_freq, rot_dims, pairing, amplitude, pos,
                      [&](int) { return ko; }, NoCopy());
    }
    return;
  }
  const int vh = hd - n_q_heads - n_k_heads;
  const float* vrow = krow + (size_t)n_k_heads * dk + (size_t)vh * dv;
  T* vo = v_cache + kv_row_offset(vp, seq, pos, vh);
  for (int e = threadIdx.x; e < dv; e += blockDim.x) vo[e] = from_f32<T>(vrow[e]);
}


template <typename T>
__global__ void __launch_bounds__(128)
qkv_prepare_heads_kernel(const float* __restrict__ proj, long ld, int n_q_heads, int n_k_heads, int dk, int n_v_heads, int dv,
                         const float* __restrict__ inv_freq, int rot_dims, int pairing, float amplitude, int v_from_k,
                         const int32_t* __restrict__ tok_seq, const int32_t* __restrict__ tok_pos, PagedKV kp, PagedKV vp,
                         T* __restrict__ k_cache, T* __restrict__ v_cache, T* __restrict__ q_out, long ldq, int write_kv,
                         int heads_per_block) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const int seq = tok_seq[t];
  const int n_all = n_q_heads + (write_kv ? n_k_heads + (v_from_k ? 0 : n_v_heads) : 0);
  for (int hd = blockIdx.y * heads_per_block; hd < min(n_all, (int)(blockIdx.y + 1) * heads_per_block); ++hd)
    prepare_head<T>(proj, ld, n_q_heads, n_k_heads, dk, dv, inv_freq, rot_dims, pairing, amplitude, v_from_k, seq, tok_pos, kp, vp,
                    k_cache, v_cache, q_out, ldq, t, hd);
}

// The same for many tokens with eight entries a thread (two 16-byte loads, one 16-byte store in bf16): neighbouring
// pairs only (a chunk of eight holds four whole pairs), sizes in multiples of eight, the values being the keys or not.
// Chunks are counted over the token's q heads, then its k heads, then its v heads; the arithmetic per entry is that of
// prepare_part.
template <typename T>
__device__ __forceinline__ void store8(T* dst, const float* v);
template <>
__device__ __forceinline__ void store8<float>(float* dst, const float* v) {
  reinterpret_cast<float4*>(dst)[0] = make_float4(v[0], v[1], v[2], v[3]);
  reinterpret_cast<float4*>(dst)[1] = make_float4(v[4], v[5], v[6], v[7]);
}
template <>
__device__ __forceinline__ void store8<__nv_bfloat16>(__nv_bfloat16* dst, const float* v) {
  __nv_bfloat162 h[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
  *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(h);
}

template <typename T>
__global__ void __launch_bounds__(128)
qkv_prepare_chunks_kernel(const float* __restrict__ proj, long ld, int n_q_heads, int n_k_heads, int dk, int n_v_heads, int dv,
                          const float* __restrict__ inv_freq, int rot_dims, float amplitude, int v_from_k,
                          const int32_t* __restrict__ tok_seq, const int32_t* __restrict__ tok_pos, PagedKV kp, PagedKV vp,
                          T* __restrict__ k_cache, T* __restrict__ v_cache, T* __restrict__ q_out, long ldq, int write_kv) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const int seq = tok_seq[t];
  const int cq = n_q_heads * dk / 8, ck = write_kv ? n_k_heads * dk / 8 : 0, cv = (write_kv && !v_from_k) ? n_v_heads * dv / 8 : 0;
  const int pos = seq >= 0 ? tok_pos[t] : 0;
  const float* row = proj + (size_t)t * ld;
  for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < cq + ck + cv; c += gridDim.y * blockDim.x) {
    float v[8];
    if (seq < 0) {
      if (c < cq) {
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] = 0.f;
        store8<T>(q_out + (size_t)t * ldq + (size_t)c * 8, v);
      }
      continue;
    }
    const float4 lo = reinterpret_cast<const float4*>(row + (size_t)c * 8)[0], hi = reinterpret_cast<const float4*>(row + (size_t)c * 8)[1];
    v[0] = lo.x; v[1] = lo.y; v[2] = lo.z; v[3] = lo.w; v[4] = hi.x; v[5] = hi.y; v[6] = hi.z; v[7] = hi.w;
    if (c >= cq + ck) {                                    // a chunk of a value head, as it is
      const int e = (c - cq - ck) * 8, hd = e / dv;
      store8<T>(v_cache + kv_row_offset(vp, seq, pos, hd) + (e - hd * dv), v);
      continue;
    }
    const int e = (c < cq ? c : c - cq) * 8, hd = e / dk, e0 = e - hd * dk;      // entries e0 .. e0 + 7 of head hd
    if (c >= cq && v_from_k) store8<T>(v_cache + kv_row_offset(vp, seq, pos, hd) + e0, v);   // the values: the keys before the rotation
    if (e0 < rot_dims) {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        float sn, cs;
        sincosf((float)pos * inv_freq[e0 / 2 + i], &sn, &cs);
        sn *= amplitude;
        cs *= amplitude;
        const float a = v[2 * i], b = v[2 * i + 1];
        v[2 * i] = rot_lo(a, b, cs, sn);
        v[2 * i + 1] = rot_hi(a, b, cs, sn);
      }
    }
    T* dst = c < cq ? q_out + (size_t)t * ldq + (size_t)hd * dk + e0 : k_cache + kv_row_offset(kp, seq, pos, hd) + e0;
    store8<T>(dst, v);
  }
}


template <typename T>
static int launch_prepare_heads(const float* proj, long ld, int n_q_heads, int n_k_heads, int dk, int n_v_heads, int dv,
                                const float* inv_freq, int rot_dims, int pairing, float amplitude, int v_from_k,
                                const int32_t* tok_seq, const int32_t* tok_pos, PagedKV kp, PagedKV vp, void* k_cache, void* v_cache,
                                void* q_out, long ldq, int n_tokens, bool kv, cudaStream_t stream) {
  const int heads = n_q_heads + (kv ? n_k_heads + (v_from_k ? 0 : n_v_heads) : 0);
  // many tokens, neighbouring pairs (or no rotation), everything in multiples of eight entries and 16 bytes: eight entries a thread
  if (n_tokens > 128 && (pairing || rot_dims == 0) && !(dk % 8) && !(dv % 8) && !(rot_dims % 8) && !(ld % 4) && !(ldq % 8) &&
      !((uintptr_t)proj & 15) && !((uintptr_t)q_out & 15) && !((uintptr_t)k_cache & 15) && !((uintptr_t)v_cache & 15)) {
    const int chunks = (n_q_heads * dk + (kv ? n_k_heads * dk + (v_from_k ? 0 : n_v_heads * dv) : 0)) / 8;
    return launch_pdl(PDL_SMALL, qkv_prepare_chunks_kernel<T>, dim3(n_tokens, (chunks + 255) / 256), dim3(128), 0, stream, proj, ld,
                      n_q_heads, n_k_heads, dk, n_v_heads, dv, inv_freq, rot_dims, amplitude, v_from_k, tok_seq, tok_pos, kp, vp,
                      (T*)k_cache, (T*)v_cache, (T*)q_out, ldq, kv ? 1 : 0);
  }
  // few tokens: a head per block of 64 threads; many: four heads per block of 128 (fewer, longer blocks)
  const int per = n_tokens <= 128 ? 1 : 4, threads = n_tokens <= 128 ? 64 : 128;
  return launch_pdl(PDL_SMALL, qkv_prepare_heads_kernel<T>, dim3(n_tokens, (heads + per - 1) / per), dim3(threads), 0, stream, proj, ld,
                    n_q_heads, n_k_heads, dk, n_v_heads, dv, inv_freq, rot_dims, pairing, amplitude, v_from_k, tok_seq, tok_pos, kp, vp,
                    (T*)k_cache, (T*)v_cache, (T*)q_out, ldq, kv ? 1 : 0, per);
}

}  // namespace llmi

using namespace llmi;

LLMI_EXPORT int llmi_qkv_prepare(int dtype, const float* proj, long ld, int n_q_heads, int n_k_heads, int dk, int n_v_heads,
                                 int dv, const float* q_norm_w, const float* k_norm_w, float eps, const float* inv_freq,
                                 int rot_dims, int pairing, float amplitude, int v_from_k, const int32_t* tok_seq,
                                 const int32_t* tok_pos, const int32_t* k_pages,
                                 int k_pages_stride, const int32_t* v_pages, int v_pages_stride, int page_size, void* k_cache,
                                 void* v_cache, void* q_out, long ldq, int n_tokens, int has_kv, int write_kv,
                                 cudaStream_t stream) {
  if (n_tokens <= 0 || n_q_heads <= 0 || dk <= 0 || page_size <= 0) return LLMI_ERR_BAD_SIZE;
  if (has_kv && (n_k_heads <= 0 || n_v_heads <= 0 || dv <= 0)) return LLMI_ERR_BAD_SIZE;
  if (rot_dims < 0 || rot_dims > dk || (rot_dims & 1) || (rot_dims > 0 && !inv_freq)) return LLMI_ERR_BAD_SIZE;
  if (v_from_k && (!has_kv || n_v_heads != n_k_heads || dv != dk)) return LLMI_ERR_BAD_SIZE;
  const PagedKV kp{k_pages, k_pages_stride, page_size, n_k_heads, dk}, vp{v_pages, v_pages_stride, page_size, n_v_heads, dv};
  if (!q_norm_w && !k_norm_w && n_q_heads + n_k_heads + n_v_heads <= 65535) {
    const bool kv = has_kv && write_kv;
    if (dtype == LLMI_DTYPE_F32)
      return launch_prepare_heads<float>(proj, ld, n_q_heads, n_k_heads, dk, n_v_heads, dv, inv_freq, rot_dims, pairing, amplitude,
                                         v_from_k, tok_seq, tok_pos, kp, vp, k_cache, v_cache, q_out, ldq, n_tokens, kv, stream);
    if (dtype == LLMI_DTYPE_BF16)
      return launch_prepare_heads<__nv_bfloat16>(proj, ld, n_q_heads, n_k_heads, dk, n_v_heads, dv, inv_freq, rot_dims, pairing,
                                                 amplitude, v_from_k, tok_seq, tok_pos, kp, vp, k_cache, v_cache, q_out, ldq, n_tokens,
                                                 kv, stream);
    return LLMI_ERR_BAD_DTYPE;
  }
  if (dtype == LLMI_DTYPE_F32)
    return launch_pdl(PDL_SMALL, qkv_prepare_kernel<float>, dim3(n_tokens), dim3(128), 0, stream, proj, ld, n_q_heads, n_k_heads,
                      dk, n_v_heads, dv, q_norm_w, k_norm_w, eps, inv_freq, rot_dims, pairing, amplitude, v_from_k, tok_seq, tok_pos, kp, vp, (float*)k_cache,
                      (float*)v_cache, (float*)q_out, ldq, has_kv, write_kv);
  if (dtype == LLMI_DTYPE_BF16)
    return launch_pdl(PDL_SMALL, qkv_prepare_kernel<__nv_bfloat16>, dim3(n_tokens), dim3(128), 0, stream, proj, ld, n_q_heads,
                      n_k_heads, dk, n_v_heads, dv, q_norm_w, k_norm_w, eps, inv_freq, rot_dims, pairing, amplitude, v_from_k, tok_seq, tok_pos, kp, vp,
                      (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache, (__nv_bfloat16*)q_out, ldq, has_kv, write_kv);
  return LLMI_ERR_BAD_DTYPE;
}
