// Causal attention over the paged cache in its general form, any sizes, fp32 arithmetic:
//   * keys and values with head sizes of their own (dk, dv) and page layouts of their own;
//   * `maps` score maps per head: query row [head][map][dk], key heads [kv head][map], all maps of a head read the
//     SAME values; the output is [head][map][dv], one softmax-weighted sum per map (what a differential
//     attention then subtracts: llmi_diff_combine);
//   * query head h reads kv head h / (heads / kv_heads);
//   * score = (q . k) * scale * head_scale[h]  (head_scale optional); with softcap > 0 the score then passes
//     softcap * tanh(score / softcap);
//   * the keys a query at position p sees: max(p - window + 1, floor(p / chunk) * chunk, 0) .. p
//     (window 0: no window; chunk 0: no chunks) — chunks are counted from position 0 of the sequence;
//   * optionally, beside a window, one pooled key and value per block of positions that lies wholly before it
//     (PooledKV below), in the same softmax, and a logistic gate on the output: one number per (token, head), or one
//     per output entry.
// One warp owns one (token, head, map).  Keys are taken 32 at a time in blocks anchored at absolute positions
// 0, 32, 64, ... with a running maximum and sum, so the order of every addition depends on the key's position only,
// not on how the step was cut or batched.  Serves prompts and single tokens of the fp32 path, and bf16 sizes that
// the tensor-core kernels do not take.
#include <math.h>

#include "common.cuh"
#include "step_meta.cuh"

namespace llmi {

constexpr int FLEX_WARPS = 4;
constexpr int FLEX_MAX_DK = 256;
constexpr int FLEX_MAX_DV = 256;

template <typename T>
__device__ __forceinline__ float flex_dot(const float* __restrict__ q, const T* __restrict__ k, int n) {
  float acc = 0.f;
  for (int d = 0; d < n; ++d) acc = fmaf(q[d], to_f32(k[d]), acc);
  return acc;
}

template <>
__device__ __forceinline__ float flex_dot<__nv_bfloat16>(const float* __restrict__ q, const __nv_bfloat16* __restrict__ k, int n) {
  float acc = 0.f;
  if ((n & 7) == 0) {
    for (int d = 0; d < n; d += 8) {
      const uint4 raw = *reinterpret_cast<const uint4*>(k + d);
      const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 f = __bfloat1622float2(p[e]);
        acc = fmaf(q[d + 2 * e], f.x, acc);
        acc = fmaf(q[d + 2 * e + 1], f.y, acc);
      }
    }
  } else {
    for (int d = 0; d < n; ++d) acc = fmaf(q[d], __bfloat162float(k[d]), acc);
  }
  return acc;
}

template <>
__device__ __forceinline__ float flex_dot<float>(const float* __restrict__ q, const float* __restrict__ k, int n) {
  float acc = 0.f;
  if ((n & 3) == 0) {
    for (int d = 0; d < n; d += 4) {
      const float4 f = *reinterpret_cast<const float4*>(k + d);
      acc = fmaf(q[d], f.x, acc);
      acc = fmaf(q[d + 1], f.y, acc);
      acc = fmaf(q[d + 2], f.z, acc);
      acc = fmaf(q[d + 3], f.w, acc);
    }
  } else {
    for (int d = 0; d < n; ++d) acc = fmaf(q[d], k[d], acc);
  }
  return acc;
}

// One run of rows lo .. hi of a paged tensor pair joins a warp's running softmax: 32 rows at a time in blocks anchored
// at multiples of 32, so the order of every addition depends on the rows' indices only.
template <typename T, int NJ>
__device__ __forceinline__ void flex_run(const float* __restrict__ q_s, const T* __restrict__ k_cache, const T* __restrict__ v_cache,
                                         const PagedKV& kp, const PagedKV& vp, int seq, int kh, int kvh, int lo, int hi, float sc,
                                         float softcap, int lane, float& m, float& l, float (&acc)[NJ]) {
  const int dk = kp.head_dim, dv = vp.head_dim;
  for (int c0 = (lo / 32) * 32; c0 <= hi; c0 += 32) {
    const int s = c0 + lane;
    const bool valid = s >= lo && s <= hi;
    float score = -INFINITY;
    if (valid) {
      score = flex_dot<T>(q_s, k_cache + kv_row_offset(kp, seq, s, kh), dk) * sc;
      if (softcap > 0.f) score = softcap * tanhf(score / softcap);
    }
    const float m_new = fmaxf(m, warp_max(score));
    const float p = valid ? expf(score - m_new) : 0.f;
    const float corr = expf(m - m_new);  // first block: exp(-inf) = 0
    l = l * corr + warp_sum(p);
#pragma unroll
    for (int j = 0; j < NJ; ++j) acc[j] *= corr;
    const int kend = (hi - c0 + 1 < 32) ? hi - c0 + 1 : 32;
    for (int kk = 0; kk < kend; ++kk) {
      const float pk = __shfl_sync(0xffffffffu, p, kk);
      if (c0 + kk < lo) continue;
      const T* vr = v_cache + kv_row_offset(vp, seq, c0 + kk, kvh);
#pragma unroll
      for (int j = 0; j < NJ; ++j) {
        const int d = lane + 32 * j;
        if (d < dv) acc[j] = fmaf(pk, to_f32(vr[d]), acc[j]);
      }
    }
    m = m_new;
  }
}

// What a query sees beside its window: rows that each sum up a block of `pool` positions (the mean of the block's keys
// and the mean of its values, kept in pages of their own).  Block b is seen once it lies wholly before the window:
// b * pool + pool - 1 <= pos - window.  The positions between the last such block and the window are not seen.
struct PooledKV {
  const void* k;       // [page][kv_heads][page_size][dk], null: none
  const void* v;
  PagedKV kp, vp;
  int pool;
};

__host__ __device__ __forceinline__ int pooled_blocks_visible(int pos, int window, int pool) {
  return (pool > 0 && window > 0 && pos - window + 1 > 0) ? (pos - window + 1) / pool : 0;
}

// NJ = ceil(dv / 32): output elements per lane.  OutT: the compute type, or float.  `gate` (optional, fp32): the
// output is multiplied by the logistic function of one number per (token, head) at gate[t * ldg + h] (gate_per 1) or of
// one number per output entry at gate[t * ldg + h * dv + d] (gate_per = dv).
template <typename T, typename OutT, int NJ>
__global__ void __launch_bounds__(FLEX_WARPS * 32)
attention_flex_kernel(const T* __restrict__ q, long ldq, OutT* __restrict__ out, long ldo, const T* __restrict__ k_cache,
                      const T* __restrict__ v_cache, const int32_t* __restrict__ tok_seq, const int32_t* __restrict__ tok_pos,
                      PagedKV kp, PagedKV vp, int n_tokens, int n_heads, int maps, float scale,
                      const float* __restrict__ head_scale, int window, int chunk, PooledKV pooled,
                      const float* __restrict__ gate, long ldg, int gate_per, float softcap) {
  __shared__ float q_s[FLEX_WARPS][FLEX_MAX_DK];
  pdl_launch_dependents();
  pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long per_tok = (long)n_heads * maps;
  const long item = (long)blockIdx.x * FLEX_WARPS + warp;
  if (item >= (long)n_tokens * per_tok) return;
  const int t = (int)(item / per_tok), hm = (int)(item - (long)t * per_tok);
  const int h = hm / maps, mp = hm - h * maps;
  const int dk = kp.head_dim, dv = vp.head_dim;
  const int seq = tok_seq[t];
  OutT* o = out + (size_t)t * ldo + (size_t)hm * dv;
  if (seq < 0) {
    for (int d = lane; d < dv; d += 32) o[d] = from_f32<OutT>(0.f);
    return;
  }
  const int pos = tok_pos[t];
  const int kvh = h / (n_heads / vp.n_kv_heads);
  const int kh = kvh * maps + mp;
  const int lo = first_visible(pos, window, chunk);
  const float sc = head_scale ? scale * head_scale[h] : scale;

  const T* qp = q + (size_t)t * ldq + (size_t)hm * dk;
  for (int d = lane; d < dk; d += 32) q_s[warp][d] = to_f32(qp[d]);
  __syncwarp();

  float m = -INFINITY, l = 0.f;
  float acc[NJ];
#pragma unroll
  for (int j = 0; j < NJ; ++j) acc[j] = 0.f;

  const int nb = pooled.k ? pooled_blocks_visible(pos, window, pooled.pool) : 0;
  if (nb > 0)
    flex_run<T, NJ>(q_s[warp], (const T*)pooled.k, (const T*)pooled.v, pooled.kp, pooled.vp, seq, kh, kvh, 0, nb - 1, sc, softcap, lane, m, l, acc);
  flex_run<T, NJ>(q_s[warp], k_cache, v_cache, kp, vp, seq, kh, kvh, lo, pos, sc, softcap, lane, m, l, acc);
  float inv = 1.0f / l;
  if (gate && gate_per <= 1) inv *= 1.0f / (1.0f + expf(-gate[(size_t)t * ldg + h]));
#pragma unroll
  for (int j = 0; j < NJ; ++j) {
    const int d = lane + 32 * j;
    if (d >= dv) continue;
    float r = acc[j] * inv;
    if (gate && gate_per > 1) r *= 1.0f / (1.0f + expf(-gate[(size_t)t * ldg + (size_t)h * dv + d]));
    o[d] = from_f32<OutT>(r);
  }
}

// Rows that sum up blocks of positions: for every token of the step whose position ends a block of `pool` positions,
// the mean of the block's `pool` key rows and of its value rows (as the cache holds them, added in position order in
// fp32) goes to row pos / pool of the pooled pages.  One block of threads per token.
template <typename T>
__global__ void __launch_bounds__(128)
pool_rows_kernel(const T* __restrict__ k_cache, const T* __restrict__ v_cache, PagedKV kp, PagedKV vp, T* __restrict__ k_pool,
                 T* __restrict__ v_pool, PagedKV kpp, PagedKV vpp, int pool, const int32_t* __restrict__ tok_seq,
                 const int32_t* __restrict__ tok_pos) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const int seq = tok_seq[t];
  if (seq < 0) return;
  const int pos = tok_pos[t];
  if ((pos + 1) % pool != 0) return;
  const int b = pos / pool, first = pos - pool + 1;
  const float inv = 1.0f / (float)pool;
  const int nk = kp.n_kv_heads * kp.head_dim, nv = vp.n_kv_heads * vp.head_dim;
  for (int idx = threadIdx.x; idx < nk + nv; idx += blockDim.x) {
    const bool is_k = idx < nk;
    const PagedKV& src = is_k ? kp : vp;
    const int i = is_k ? idx : idx - nk;
    const int hd = i / src.head_dim, e = i - hd * src.head_dim;
    const T* cache = is_k ? k_cache : v_cache;
    float sum = 0.f;
    for (int j = 0; j < pool; ++j) sum += to_f32(cache[kv_row_offset(src, seq, first + j, hd) + e]);
    if (is_k) k_pool[kv_row_offset(kpp, seq, b, hd) + e] = from_f32<T>(sum * inv);
    else v_pool[kv_row_offset(vpp, seq, b, hd) + e] = from_f32<T>(sum * inv);
  }
}

// The same for bf16 rows of whole 16-byte pieces: a thread owns one piece (8 entries) of a head's row and adds the
// block's rows in position order; blockIdx.y cuts the pieces of a row over several blocks.
__global__ void __launch_bounds__(128)
pool_rows_vec_kernel(const __nv_bfloat16* __restrict__ k_cache, const __nv_bfloat16* __restrict__ v_cache, PagedKV kp, PagedKV vp,
                     __nv_bfloat16* __restrict__ k_pool, __nv_bfloat16* __restrict__ v_pool, PagedKV kpp, PagedKV vpp, int pool,
                     const int32_t* __restrict__ tok_seq, const int32_t* __restrict__ tok_pos) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const int seq = tok_seq[t];
  if (seq < 0) return;
  const int pos = tok_pos[t];
  if ((pos + 1) % pool != 0) return;
  const int b = pos / pool, first = pos - pool + 1;
  const float inv = 1.0f / (float)pool;
  const int nk = kp.n_kv_heads * kp.head_dim / 8, nv = vp.n_kv_heads * vp.head_dim / 8;
  for (int idx = blockIdx.y * blockDim.x + threadIdx.x; idx < nk + nv; idx += gridDim.y * blockDim.x) {
    const bool is_k = idx < nk;
    const PagedKV& src = is_k ? kp : vp;
    const int i = is_k ? idx : idx - nk;
    const int per = src.head_dim / 8;
    const int hd = i / per, e = (i - hd * per) * 8;
    const __nv_bfloat16* cache = is_k ? k_cache : v_cache;
    float sum[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll 4
    for (int j = 0; j < pool; ++j) {
      const uint4 u = *reinterpret_cast<const uint4*>(cache + kv_row_offset(src, seq, first + j, hd) + e);
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
      for (int x = 0; x < 4; ++x) {
        const float2 f = __bfloat1622float2(h[x]);
        sum[2 * x] += f.x;
        sum[2 * x + 1] += f.y;
      }
    }
    uint4 o;
    __nv_bfloat162* oh = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
    for (int x = 0; x < 4; ++x) oh[x] = __floats2bfloat162_rn(sum[2 * x] * inv, sum[2 * x + 1] * inv);
    __nv_bfloat16* dst = is_k ? k_pool + kv_row_offset(kpp, seq, b, hd) + e : v_pool + kv_row_offset(vpp, seq, b, hd) + e;
    *reinterpret_cast<uint4*>(dst) = o;
  }
}

template <typename T, typename OutT>
int launch_attention_flex(const void* q, long ldq, void* out, long ldo, const void* k_cache, const void* v_cache,
                          const int32_t* tok_seq, const int32_t* tok_pos, PagedKV kp, PagedKV vp, int n_tokens, int n_heads,
                          int maps, float scale, const float* head_scale, int window, int chunk, PooledKV pooled,
                          const float* gate, long ldg, int gate_per, float softcap, cudaStream_t stream) {
  const long items = (long)n_tokens * n_heads * maps;
  const long blocks = (items + FLEX_WARPS - 1) / FLEX_WARPS;
  if (blocks > 0x7fffffffL) return LLMI_ERR_BAD_SIZE;
  const int nj = (vp.head_dim + 31) / 32;
#define LLMI_LAUNCH(NJ)                                                                                                  \
  return launch_pdl(PDL_ATTENTION, attention_flex_kernel<T, OutT, NJ>, dim3((unsigned)blocks), dim3(FLEX_WARPS * 32), 0, \
                    stream, (const T*)q, ldq, (OutT*)out, ldo, (const T*)k_cache, (const T*)v_cache, tok_seq, tok_pos,   \
                    kp, vp, n_tokens, n_heads, maps, scale, head_scale, window, chunk, pooled, gate, ldg, gate_per, softcap)
  if (nj <= 1) LLMI_LAUNCH(1);
  if (nj <= 2) LLMI_LAUNCH(2);
  if (nj <= 4) LLMI_LAUNCH(4);
  LLMI_LAUNCH(8);
#undef LLMI_LAUNCH
}

// Differential attention's join: per (token, head), from the two maps' outputs a1, a2 (fp32, [head][2][dv]):
//   o = a1 - lambda * a2;   o <- o / sqrt(mean(o^2) + eps) * post     (no weight), in the compute type.
template <typename T>
__global__ void __launch_bounds__(128)
diff_combine_kernel(const float* __restrict__ a, long lda, float lambda, float eps, float post, int H, int dv,
                    const int32_t* __restrict__ tok_seq, T* __restrict__ out, long ldo, long n_items) {
  pdl_launch_dependents();
  pdl_wait();
  const long item = (long)blockIdx.x * 4 + (threadIdx.x >> 5);
  if (item >= n_items) return;
  const int lane = threadIdx.x & 31;
  const int t = (int)(item / H), h = (int)(item - (long)t * H);
  T* dst = out + (size_t)t * ldo + (size_t)h * dv;
  if (tok_seq[t] < 0) {
    for (int d = lane; d < dv; d += 32) dst[d] = from_f32<T>(0.f);
    return;
  }
  const float* a1 = a + (size_t)t * lda + (size_t)h * 2 * dv;
  const float* a2 = a1 + dv;
  float ss = 0.f;
  for (int d = lane; d < dv; d += 32) {
    const float o = fmaf(-lambda, a2[d], a1[d]);
    ss = fmaf(o, o, ss);
  }
  ss = warp_sum(ss);
  const float sc = post / sqrtf(ss / (float)dv + eps);
  for (int d = lane; d < dv; d += 32) dst[d] = from_f32<T>(fmaf(-lambda, a2[d], a1[d]) * sc);
}

}  // namespace llmi

using namespace llmi;

// q [T, >= heads*maps*dk] (row-strided) in `dtype`; out [T, heads*maps*dv] in `dtype`, or fp32 if out_f32.
LLMI_EXPORT int llmi_attention_flex(int dtype, const void* q, long ldq, void* out, long ldo, int out_f32, const void* k_cache,
                                    const void* v_cache, const int32_t* tok_seq, const int32_t* tok_pos,
                                    const int32_t* seq_pages, int pages_stride, int page_size, int n_tokens, int n_heads,
                                    int n_kv_heads, int maps, int dk, int dv, float scale, const float* head_scale, int window,
                                    int chunk, int pool, const void* k_pool, const void* v_pool, const int32_t* pool_pages,
                                    int pool_pages_stride, const float* gate, long ldg, int gate_per, float softcap,
                                    cudaStream_t stream) {
  if (n_tokens <= 0 || n_heads <= 0 || n_kv_heads <= 0 || maps <= 0 || dk <= 0 || dv <= 0 || page_size <= 0) return LLMI_ERR_BAD_SIZE;
  if (gate && gate_per != 1 && (gate_per != dv || maps != 1)) return LLMI_ERR_UNSUPPORTED;
  if (softcap < 0.f) return LLMI_ERR_BAD_SIZE;
  if (dk > FLEX_MAX_DK || dv > FLEX_MAX_DV || n_heads % n_kv_heads != 0 || window < 0 || chunk < 0) return LLMI_ERR_BAD_SIZE;
  if (pool < 0 || (pool > 0 && (!k_pool || !v_pool || !pool_pages || window <= 0))) return LLMI_ERR_BAD_SIZE;
  const PagedKV kp{seq_pages, pages_stride, page_size, n_kv_heads * maps, dk}, vp{seq_pages, pages_stride, page_size, n_kv_heads, dv};
  PooledKV pooled{pool > 0 ? k_pool : nullptr, pool > 0 ? v_pool : nullptr,
                  PagedKV{pool_pages, pool_pages_stride, page_size, n_kv_heads * maps, dk},
                  PagedKV{pool_pages, pool_pages_stride, page_size, n_kv_heads, dv}, pool};
#define LLMI_ARGS q, ldq, out, ldo, k_cache, v_cache, tok_seq, tok_pos, kp, vp, n_tokens, n_heads, maps, scale, head_scale, window, chunk, pooled, gate, ldg, gate_per, softcap, stream
  if (dtype == LLMI_DTYPE_F32) return launch_attention_flex<float, float>(LLMI_ARGS);
  if (dtype == LLMI_DTYPE_BF16)
    return out_f32 ? launch_attention_flex<__nv_bfloat16, float>(LLMI_ARGS) : launch_attention_flex<__nv_bfloat16, __nv_bfloat16>(LLMI_ARGS);
#undef LLMI_ARGS
  return LLMI_ERR_BAD_DTYPE;
}

// For every token of the step that ends a block of `pool` positions: the block's mean key and value rows (see
// pool_rows_kernel).  The token pages and the pooled pages have page tables of their own.
LLMI_EXPORT int llmi_pool_rows(int dtype, const void* k_cache, const void* v_cache, const int32_t* seq_pages, int pages_stride,
                               void* k_pool, void* v_pool, const int32_t* pool_pages, int pool_pages_stride, int page_size,
                               int n_k_heads, int dk, int n_v_heads, int dv, int pool, const int32_t* tok_seq,
                               const int32_t* tok_pos, int n_tokens, cudaStream_t stream) {
  if (n_tokens <= 0 || pool <= 0 || n_k_heads <= 0 || n_v_heads <= 0 || dk <= 0 || dv <= 0 || page_size <= 0) return LLMI_ERR_BAD_SIZE;
  const PagedKV kp{seq_pages, pages_stride, page_size, n_k_heads, dk}, vp{seq_pages, pages_stride, page_size, n_v_heads, dv};
  const PagedKV kpp{pool_pages, pool_pages_stride, page_size, n_k_heads, dk}, vpp{pool_pages, pool_pages_stride, page_size, n_v_heads, dv};
  if (dtype == LLMI_DTYPE_F32)
    return launch_pdl(PDL_SMALL, pool_rows_kernel<float>, dim3(n_tokens), dim3(128), 0, stream, (const float*)k_cache,
                      (const float*)v_cache, kp, vp, (float*)k_pool, (float*)v_pool, kpp, vpp, pool, tok_seq, tok_pos);
  if (dtype == LLMI_DTYPE_BF16 && dk % 8 == 0 && dv % 8 == 0 && !((uintptr_t)k_cache & 15) && !((uintptr_t)v_cache & 15) &&
      !((uintptr_t)k_pool & 15) && !((uintptr_t)v_pool & 15)) {
    const int pieces = (n_k_heads * dk + n_v_heads * dv) / 8;
    const int cuts = n_tokens <= 64 ? (pieces + 127) / 128 : 1;       // few tokens: a row's pieces over several blocks
    return launch_pdl(PDL_SMALL, pool_rows_vec_kernel, dim3(n_tokens, cuts), dim3(128), 0, stream, (const __nv_bfloat16*)k_cache,
                      (const __nv_bfloat16*)v_cache, kp, vp, (__nv_bfloat16*)k_pool, (__nv_bfloat16*)v_pool, kpp, vpp, pool, tok_seq,
                      tok_pos);
  }
  if (dtype == LLMI_DTYPE_BF16)
    return launch_pdl(PDL_SMALL, pool_rows_kernel<__nv_bfloat16>, dim3(n_tokens), dim3(128), 0, stream, (const __nv_bfloat16*)k_cache,
                      (const __nv_bfloat16*)v_cache, kp, vp, (__nv_bfloat16*)k_pool, (__nv_bfloat16*)v_pool, kpp, vpp, pool, tok_seq,
                      tok_pos);
  return LLMI_ERR_BAD_DTYPE;
}

LLMI_EXPORT int llmi_diff_combine(int dtype, const float* a, long lda, float lambda, float eps, float post, int H, int dv,
                                  const int32_t* tok_seq, void* out, long ldo, int n_tokens, cudaStream_t stream) {
  if (n_tokens <= 0 || H <= 0 || dv <= 0) return LLMI_ERR_BAD_SIZE;
  const long items = (long)n_tokens * H;
  const unsigned blocks = (unsigned)((items + 3) / 4);
  if (dtype == LLMI_DTYPE_F32)
    return launch_pdl(PDL_SMALL, diff_combine_kernel<float>, dim3(blocks), dim3(128), 0, stream, a, lda, lambda, eps, post, H, dv,
                      tok_seq, (float*)out, ldo, items);
  if (dtype == LLMI_DTYPE_BF16)
    return launch_pdl(PDL_SMALL, diff_combine_kernel<__nv_bfloat16>, dim3(blocks), dim3(128), 0, stream, a, lda, lambda, eps, post,
                      H, dv, tok_seq, (__nv_bfloat16*)out, ldo, items);
  return LLMI_ERR_BAD_DTYPE;
}
