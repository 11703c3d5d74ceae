// Attention in its general form on the tensor cores (bf16): keys and values with head sizes of their own, `maps`
// score maps per head over one set of values, a factor per head on the scores, a window and a mask of blocks of
// positions.  The same meaning as attention_flex.cu; sizes: dk, dv multiples of 16 up to 128, pages of 64 positions.
//
// Flash style with mma.sync m16n8k16 (bf16 in, fp32 out): a warp holds 16 query rows; S = Q Kᵀ from shared memory by
// ldmatrix; the softmax runs on the accumulators with a running maximum and sum per row (fp32, base 2 with the scale
// folded in); P goes back in as the A operand of O += P V straight from the registers it was computed in.  K and V
// pages arrive by cp.async into two buffers, the next page while the current one is
// multiplied; value rows beyond a sequence's newest position arrive as zeros (their weights are zero, and 0 x anything
// must stay 0).
//
// Two forms of one kernel:
//   prompts        a block is 128 consecutive tokens of one sequence and one (head, map): eight warps of 16 rows each,
//                  every warp multiplies all 64 keys of a page; the result leaves normalised.  Blocks of later rows
//                  (longer key ranges) come first in the grid.
//   single tokens  a block is one (sequence, kv head, map, cut over the positions): its 16 rows are the query heads
//                  that share the kv head, every warp takes 16 of a page's 64 keys with a running state of its own;
//                  the four states meet in shared memory in warp order, and the block leaves (maximum, sum,
//                  unnormalised O) per row in a workspace, one part per cut, which a second kernel joins in a fixed
//                  order — or the finished row, when the positions are not cut.
// Optionally (pool > 0, beside a window) a query also sees one pooled key and value per block of `pool` positions that
// lies wholly before its window: rows of pages of their own (one row per block), walked as further 64-row tiles AHEAD of
// the window's pages in the same loop and the same running softmax; and optionally every head's output is multiplied by
// the logistic function of a number per (token, head), or every output entry by that of a number of its own; and
// optionally (softcap > 0) a score passes softcap * tanh(score / softcap) before the softmax.
// The order of every addition depends on positions only (pages anchored at multiples of 64, parts by key index), not
// on the batch; cuts follow the page table's width, which is part of a recorded step's shape.
#include <math.h>

#include "common.cuh"
#include "mma_sync.cuh"
#include "step_meta.cuh"

namespace llmi {

constexpr int AM_PAGE = 64, AM_WARPS = 4, AM_PAD = 8;      // AM_WARPS: of the form for single tokens
constexpr int AM_PROMPT_WARPS = 8, AM_PROMPT_ROWS = 16 * AM_PROMPT_WARPS;
// Page buffers of the form for single tokens.  Measured, a decode step at batch 8 and 4,096 positions: 0.585 ms with two
// buffers (four blocks fit an SM), 0.600 with three (two pages under way a block, but three blocks an SM); batch 1:
// 1,899 against 1,915 tokens/s.
constexpr int AM_TOKEN_BUFFERS = 2;

struct MapsArgs {
  const __nv_bfloat16* q;       // [T, heads, maps, dk]
  long ldq;
  void* out;                    // [T, heads, maps, dv], bf16 or fp32
  long ldo;
  int out_f32;
  const __nv_bfloat16* k_cache; // [page][kv_heads * maps][64][dk]
  const __nv_bfloat16* v_cache; // [page][kv_heads][64][dv]
  const int32_t* tok_seq;
  const int32_t* tok_pos;
  const int32_t* seq_pages;
  int pages_stride;
  const int32_t* seq_q_start;
  const int32_t* seq_kv_len;
  int n_seqs, H, G, maps, dk;
  float scale_log2;             // scale * log2(e)
  const float* head_scale;      // [H] or null
  int window, chunk;
  int splits, pages_per_split;  // single tokens
  float* ws_o;                  // [T * H * maps][splits][dv]
  float* ws_ml;                 // [T * H * maps][splits][2]
  int pool;                     // positions per pooled block (0: none)
  const __nv_bfloat16* k_pool;  // [page][kv_heads * maps][64][dk], one row per block
  const __nv_bfloat16* v_pool;  // [page][kv_heads][64][dv]
  const int32_t* pool_pages;    // [n_seqs, pool_pages_stride]
  int pool_pages_stride;
  const float* gate;            // [T, ldg]: head h's output times logistic(gate[t * ldg + h]); null: none
  long ldg;
  int gate_per;                 // 1: a number per head; dv: a number per output entry, at gate[t * ldg + h * dv + d] (one map)
  float softcap_log2;           // softcap * log2(e); 0: scores are not capped
};

__device__ __forceinline__ int maps_pooled_visible(int pos, int window, int pool) {
  return (pool > 0 && window > 0 && pos - window + 1 > 0) ? (pos - window + 1) / pool : 0;
}
__device__ __forceinline__ float maps_gate(const MapsArgs& a, int t, int head) {
  return (a.gate && a.gate_per <= 1) ? 1.0f / (1.0f + __expf(-a.gate[(size_t)t * a.ldg + head])) : 1.0f;
}
// the gate of one output entry (1 where the gate is a number per head: maps_gate has it)
__device__ __forceinline__ float maps_gate_entry(const MapsArgs& a, int t, int head, int dv, int d) {
  return (a.gate && a.gate_per > 1) ? 1.0f / (1.0f + __expf(-a.gate[(size_t)t * a.ldg + (size_t)head * dv + d])) : 1.0f;
}
// tanh on the exponential unit: 1 - 2 / (1 + e^(2x)); x is a score over its cap, the result ends up in a bf16 weight
__device__ __forceinline__ float maps_tanh(float x) { return 1.0f - __fdividef(2.0f, 1.0f + __expf(2.0f * x)); }

// NV = dv / 16.  PROMPT: the form (see above).
template <int NV, bool PROMPT>
__global__ void __launch_bounds__((PROMPT ? AM_PROMPT_WARPS : AM_WARPS) * 32)
attention_maps_mma_kernel(const MapsArgs a) {
  extern __shared__ __align__(16) unsigned char am_smem[];
  pdl_wait();
  pdl_launch_dependents();
  constexpr int DV = NV * 16, ROWS = PROMPT ? AM_PROMPT_ROWS : 16, NT2 = PROMPT ? 4 : 1;
  constexpr int NBUF = PROMPT ? 2 : AM_TOKEN_BUFFERS;             // page buffers: NBUF - 1 pages are under way while one is multiplied     // NT2: groups of 16 keys a warp takes per page
  const int dk = a.dk, ldk = dk + AM_PAD, ldv = DV + AM_PAD;
  __nv_bfloat16* q_s = reinterpret_cast<__nv_bfloat16*>(am_smem);                // [ROWS][ldk]
  __nv_bfloat16* k_s = q_s + ROWS * ldk;                                          // [NBUF][64][ldk]
  __nv_bfloat16* v_s = k_s + NBUF * AM_PAGE * ldk;                                // [NBUF][64][ldv]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, tq = lane & 3;
  const int group = a.H / a.G;

  int seq, t0, n_rows, kvh, mp, split = 0, head0;
  if (PROMPT) {
    int blk = blockIdx.x;
    seq = -1;
    for (int s = 0; s < a.n_seqs; ++s) {
      const int len = a.seq_q_start[s + 1] - a.seq_q_start[s];
      const int nb = len > 0 ? (len + ROWS - 1) / ROWS : 0;
      if (blk < nb) { seq = s; blk = nb - 1 - blk; break; }      // later rows first: they have the longest key ranges
      blk -= nb;
    }
    if (seq < 0) return;
    const int start = a.seq_q_start[seq], len = a.seq_q_start[seq + 1] - start;
    t0 = start + ROWS * blk;
    n_rows = min(ROWS, len - ROWS * blk);
    head0 = blockIdx.y / a.maps;
    mp = blockIdx.y - head0 * a.maps;
    kvh = head0 / group;
  } else {
    seq = blockIdx.x;
    t0 = a.seq_q_start[seq];
    n_rows = 1;
    kvh = blockIdx.y / a.maps;
    mp = blockIdx.y - kvh * a.maps;
    head0 = kvh * group;
    split = blockIdx.z;
    if (a.seq_kv_len[seq] <= 0 || a.tok_seq[t0] < 0) {
      if (a.splits == 1)                                        // a sequence of no token: zeros (with cuts, the joining kernel writes them)
        for (int idx = threadIdx.x; idx < group * (NV * 16); idx += blockDim.x) {
          const size_t at = (size_t)t0 * a.ldo + ((size_t)(head0 + idx / (NV * 16)) * a.maps + mp) * (NV * 16) + idx % (NV * 16);
          if (a.out_f32) ((float*)a.out)[at] = 0.f;
          else ((__nv_bfloat16*)a.out)[at] = __float2bfloat16_rn(0.f);
        }
      return;
    }
  }
  if (a.tok_seq[t0] < 0) return;
  const int newest = a.seq_kv_len[seq] - 1;
  const int p_first = a.tok_pos[t0], p_last = p_first + n_rows - 1;
  const int lo_first = first_visible(p_first, a.window, a.chunk);

  // queries into shared memory; rows of no token (or of no head) are zeros
  const int chunks_k = dk / 8;
  for (int idx = threadIdx.x; idx < ROWS * chunks_k; idx += blockDim.x) {
    const int r = idx / chunks_k, c8 = idx - r * chunks_k;
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (PROMPT) {
      if (r < n_rows) v = *reinterpret_cast<const uint4*>(a.q + (size_t)(t0 + r) * a.ldq + (size_t)(head0 * a.maps + mp) * dk + 8 * c8);
    } else {
      if (r < group) v = *reinterpret_cast<const uint4*>(a.q + (size_t)t0 * a.ldq + (size_t)((head0 + r) * a.maps + mp) * dk + 8 * c8);
    }
    *reinterpret_cast<uint4*>(q_s + r * ldk + 8 * c8) = v;
  }

  // my two rows (g and g + 8 of my warp's 16): position, first visible key, pooled blocks it sees, factor on the scores
  int row_pos[2], row_lo[2], row_nb[2];
  float row_scale[2];
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int r = (PROMPT ? 16 * warp : 0) + g + 8 * i;
    const bool ok = PROMPT ? r < n_rows : r < group;
    row_pos[i] = ok ? (PROMPT ? p_first + r : p_first) : -1;
    row_lo[i] = ok ? first_visible(row_pos[i], a.window, a.chunk) : 0;
    row_nb[i] = ok ? maps_pooled_visible(row_pos[i], a.window, a.pool) : 0;
    const int head = PROMPT ? head0 : head0 + (ok ? r : 0);
    row_scale[i] = a.head_scale ? a.scale_log2 * a.head_scale[head] : a.scale_log2;
  }
  // what my warp's rows can see at all (a page outside costs my warp nothing)
  int w_hi, w_lo;
  if (PROMPT) {
    const int r_lo = 16 * warp, r_hi = min(16 * warp + 15, n_rows - 1);
    w_hi = r_lo < n_rows ? p_first + r_hi : -1;
    w_lo = r_lo < n_rows ? first_visible(p_first + r_lo, a.window, a.chunk) : 0;
  } else {
    w_hi = p_first;
    w_lo = lo_first;
  }

  // The tiles the block walks, numbered from 0: first the pooled pages that its rows see (n_pp of them), then the
  // window's pages tpg_lo ..; `pg` below is this number.
  const int w_nb = maps_pooled_visible(w_hi, a.window, a.pool);            // pooled blocks my warp's rows see at most
  const int n_pool_rows = a.pool > 0 ? (newest + 1) / a.pool : 0;          // pooled rows the sequence holds
  const int n_pp = (maps_pooled_visible(p_last, a.window, a.pool) + AM_PAGE - 1) / AM_PAGE;
  const int tpg_lo = lo_first / AM_PAGE;
  int pg_lo = 0, pg_hi = n_pp + (p_last / AM_PAGE - tpg_lo);
  if (!PROMPT) {
    pg_lo += split * a.pages_per_split;
    pg_hi = min(pg_hi, pg_lo + a.pages_per_split - 1);
  }
  const int kh = kvh * a.maps + mp;
  const int chunks_v = DV / 8;
  // my first 16-byte piece of a key tile and the step from one of my pieces to the next (no division per piece)
  const int kr0 = threadIdx.x / chunks_k, kc0 = threadIdx.x - kr0 * chunks_k;
  const int kr_step = blockDim.x / chunks_k, kc_step = blockDim.x - kr_step * chunks_k;
  auto page_of = [&](int pg) {
    if (pg > pg_hi) return -1;
    return pg < n_pp ? a.pool_pages[(size_t)seq * a.pool_pages_stride + pg] : a.seq_pages[(size_t)seq * a.pages_stride + tpg_lo + pg - n_pp];
  };
  // `page`: the page's index in the cache, read from the table one iteration ahead of its copies
  auto fetch = [&](int pg, int buf, int page) {
    const bool pooled = pg < n_pp;
    const __nv_bfloat16* ksrc = (pooled ? a.k_pool : a.k_cache) + ((size_t)(page < 0 ? 0 : page) * (a.G * a.maps) + kh) * AM_PAGE * dk;
    const __nv_bfloat16* vsrc = (pooled ? a.v_pool : a.v_cache) + ((size_t)(page < 0 ? 0 : page) * a.G + kvh) * AM_PAGE * DV;
    __nv_bfloat16* kd = k_s + (size_t)buf * AM_PAGE * ldk;
    __nv_bfloat16* vd = v_s + (size_t)buf * AM_PAGE * ldv;
    // rows of the page that hold a position (or a finished block)
    const int live_rows = page < 0 ? 0 : pooled ? n_pool_rows - pg * AM_PAGE : newest - (tpg_lo + pg - n_pp) * AM_PAGE + 1;
    for (int r = kr0, c8 = kc0; r < AM_PAGE;) {
      const bool live = r < live_rows;
      cp_async16(kd + r * ldk + 8 * c8, live ? ksrc + (size_t)r * dk + 8 * c8 : a.k_cache, live ? 16 : 0);
      r += kr_step;
      c8 += kc_step;
      if (c8 >= chunks_k) { c8 -= chunks_k; ++r; }
    }
    for (int idx = threadIdx.x; idx < AM_PAGE * chunks_v; idx += blockDim.x) {
      const int r = idx / chunks_v, c8 = idx - r * chunks_v;
      const bool live = r < live_rows;
      cp_async16(vd + r * ldv + 8 * c8, live ? vsrc + (size_t)r * DV + 8 * c8 : a.v_cache, live ? 16 : 0);
    }
    cp_async_commit();
  };

  const float inv_cap = a.softcap_log2 > 0.f ? 1.0f / a.softcap_log2 : 0.f;
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
  float o[2 * NV][4];
#pragma unroll
  for (int j = 0; j < 2 * NV; ++j)
#pragma unroll
    for (int e = 0; e < 4; ++e) o[j][e] = 0.f;

#pragma unroll
  for (int ahead = 0; ahead < NBUF - 1; ++ahead) {               // (a group per page, also an empty one: the waits count groups)
    if (pg_lo + ahead <= pg_hi) fetch(pg_lo + ahead, ahead, page_of(pg_lo + ahead));
    else cp_async_commit();
  }
  int page_next = page_of(pg_lo + NBUF - 1);
  const int key_off = PROMPT ? 0 : 16 * warp;                    // my keys within a page
  const __nv_bfloat16* a_ptr = q_s + ((PROMPT ? 16 * warp : 0) + (lane & 15)) * ldk + (lane >> 4) * 8;
  for (int pg = pg_lo; pg <= pg_hi; ++pg) {
    const int buf = (pg - pg_lo) % NBUF;
    cp_async_wait<NBUF - 2>();
    __syncthreads();                                             // this page is here; everyone is done with the page before
    if (pg + NBUF - 1 <= pg_hi) fetch(pg + NBUF - 1, (pg - pg_lo + NBUF - 1) % NBUF, page_next);
    else cp_async_commit();
    page_next = page_of(pg + NBUF);
    const bool pooled = pg < n_pp;
    const int base = (pooled ? pg : tpg_lo + pg - n_pp) * AM_PAGE + key_off;     // the first of my keys: a block's or a position's index
    if (pooled ? base >= w_nb : (base > w_hi || base + 16 * NT2 - 1 < w_lo)) continue;     // nothing here for my rows
    const __nv_bfloat16* kt = k_s + (size_t)buf * AM_PAGE * ldk;
    const __nv_bfloat16* vt = v_s + (size_t)buf * AM_PAGE * ldv;

    float s[2 * NT2][4];
#pragma unroll
    for (int j = 0; j < 2 * NT2; ++j)
#pragma unroll
      for (int e = 0; e < 4; ++e) s[j][e] = 0.f;
    const __nv_bfloat16* b_ptr = kt + (key_off + (lane >> 4) * 8 + (lane & 7)) * ldk + ((lane >> 3) & 1) * 8;
    for (int k0 = 0; k0 < dk; k0 += 16) {
      uint32_t af[4];
      ldsm_x4(af, a_ptr + k0);
#pragma unroll
      for (int c = 0; c < NT2; ++c) {
        uint32_t bf[4];
        ldsm_x4(bf, b_ptr + (size_t)16 * c * ldk + k0);
        mma_bf16(s[2 * c], af, bf[0], bf[1]);
        mma_bf16(s[2 * c + 1], af, bf[2], bf[3]);
      }
    }
    // scale, mask, and the maximum of each of my rows over my keys
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int j = 0; j < 2 * NT2; ++j)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int key = base + 8 * j + 2 * tq + (e & 1), i = e >> 1;
        const bool seen = pooled ? key < row_nb[i] : (key <= row_pos[i] && key >= row_lo[i]);
        float v = seen ? s[j][e] * row_scale[i] : -INFINITY;
        if (a.softcap_log2 > 0.f && seen) v = a.softcap_log2 * maps_tanh(v * inv_cap);
        s[j][e] = v;
        mx[i] = fmaxf(mx[i], v);
      }
    float corr[2], shift[2], ps[2] = {0.f, 0.f};
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 1));
      mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 2));
      const float m_new = fmaxf(m_run[i], mx[i]);
      corr[i] = m_new == -INFINITY ? 1.f : fast_exp2(m_run[i] - m_new);        // a row that has seen no key yet keeps its zeros
      shift[i] = m_new == -INFINITY ? 0.f : m_new;
      m_run[i] = m_new;
    }
    uint32_t pa[NT2][4];
#pragma unroll
    for (int c = 0; c < NT2; ++c)
#pragma unroll
      for (int jj = 0; jj < 2; ++jj)
#pragma unroll
        for (int i = 0; i < 2; ++i) {
          const int j = 2 * c + jj;
          const __nv_bfloat162 pp = __floats2bfloat162_rn(fast_exp2(s[j][2 * i] - shift[i]), fast_exp2(s[j][2 * i + 1] - shift[i]));
          ps[i] += __low2float(pp) + __high2float(pp);                       // the sum runs over the rounded weights
          pa[c][2 * jj + i] = *reinterpret_cast<const uint32_t*>(&pp);
        }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      ps[i] += __shfl_xor_sync(0xffffffffu, ps[i], 1);
      ps[i] += __shfl_xor_sync(0xffffffffu, ps[i], 2);
      l_run[i] = l_run[i] * corr[i] + ps[i];
    }
#pragma unroll
    for (int j = 0; j < 2 * NV; ++j) {
      o[j][0] *= corr[0]; o[j][1] *= corr[0];
      o[j][2] *= corr[1]; o[j][3] *= corr[1];
    }
    const __nv_bfloat16* v_ptr = vt + (key_off + ((lane >> 3) & 1) * 8 + (lane & 7)) * ldv + (lane >> 4) * 8;
#pragma unroll
    for (int c = 0; c < NT2; ++c)
#pragma unroll
      for (int j = 0; j < 2 * NV; j += 2) {
        uint32_t bf[4];
        ldsm_x4_t(bf, v_ptr + (size_t)16 * c * ldv + 8 * j);
        mma_bf16(o[j], pa[c], bf[0], bf[1]);
        mma_bf16(o[j + 1], pa[c], bf[2], bf[3]);
      }
  }
  cp_async_wait_all();

#pragma unroll
  for (int i = 0; i < 2; ++i) {
    if (!PROMPT || row_pos[i] < 0) continue;
    {
      const int t = t0 + 16 * warp + g + 8 * i;
      const float inv = maps_gate(a, t, head0) / l_run[i];
      const size_t at = (size_t)t * a.ldo + (size_t)(head0 * a.maps + mp) * DV + 2 * tq;
#pragma unroll
      for (int j = 0; j < 2 * NV; ++j) {
        const float r0 = o[j][2 * i] * inv * maps_gate_entry(a, t, head0, DV, 8 * j + 2 * tq);
        const float r1 = o[j][2 * i + 1] * inv * maps_gate_entry(a, t, head0, DV, 8 * j + 2 * tq + 1);
        if (a.out_f32) *reinterpret_cast<float2*>((float*)a.out + at + 8 * j) = make_float2(r0, r1);
        else *reinterpret_cast<__nv_bfloat162*>((__nv_bfloat16*)a.out + at + 8 * j) = __floats2bfloat162_rn(r0, r1);
      }
    }
  }
  if (!PROMPT) {
    // The four warps' states (each over its quarter of every page's keys) meet in shared memory, in warp order: the
    // block leaves ONE (maximum, sum, O) per row — or, when the positions are not cut, the finished row.
    constexpr int PW = DV + 2;
    float* part_s = reinterpret_cast<float*>(v_s);             // [4][16][DV + 2]: fits the value buffers
    __syncthreads();                                           // everyone is done with the last page
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      float* dst = part_s + (size_t)(warp * 16 + g + 8 * i) * PW;
#pragma unroll
      for (int j = 0; j < 2 * NV; ++j) *reinterpret_cast<float2*>(dst + 8 * j + 2 * tq) = make_float2(o[j][2 * i], o[j][2 * i + 1]);
      if (tq == 0) {
        dst[DV] = m_run[i];
        dst[DV + 1] = l_run[i];
      }
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < group * DV; idx += blockDim.x) {
      const int r = idx / DV, c = idx - r * DV;
      float M = -INFINITY;
#pragma unroll
      for (int w = 0; w < AM_WARPS; ++w) M = fmaxf(M, part_s[(size_t)(w * 16 + r) * PW + DV]);
      float acc = 0.f, l = 0.f;
#pragma unroll
      for (int w = 0; w < AM_WARPS; ++w) {
        const float* src = part_s + (size_t)(w * 16 + r) * PW;
        const float wt = src[DV] == -INFINITY ? 0.f : exp2f(src[DV] - M);
        acc = fmaf(wt, src[c], acc);
        l = fmaf(wt, src[DV + 1], l);
      }
      const size_t hm = (size_t)(head0 + r) * a.maps + mp;
      if (a.splits == 1) {
        const size_t at = (size_t)t0 * a.ldo + hm * DV + c;
        const float res = acc / l * maps_gate(a, t0, head0 + r) * maps_gate_entry(a, t0, head0 + r, DV, c);
        if (a.out_f32) ((float*)a.out)[at] = res;
        else ((__nv_bfloat16*)a.out)[at] = __float2bfloat16_rn(res);
      } else {
        const size_t part = ((size_t)t0 * a.H * a.maps + hm) * a.splits + split;
        a.ws_o[part * DV + c] = acc;
        if (c == 0) {
          a.ws_ml[2 * part] = M;
          a.ws_ml[2 * part + 1] = l;
        }
      }
    }
  }
}

// One block per (token, head, map): joins the parts in their order.  out = sum_p 2^(m_p - M) O_p / sum_p 2^(m_p - M) l_p.
constexpr int AM_MAX_PARTS = 1024;
__global__ void __launch_bounds__(128)
attention_maps_join_kernel(const float* __restrict__ ws_o, const float* __restrict__ ws_ml, void* __restrict__ out, long ldo,
                           int out_f32, const int32_t* __restrict__ tok_seq, int per_tok, int dv, int parts,
                           const float* __restrict__ gate, long ldg, int maps, int gate_per) {
  __shared__ float w_s[AM_MAX_PARTS];
  __shared__ float red[32];
  pdl_wait();
  pdl_launch_dependents();
  const long item = blockIdx.x;
  const int t = (int)(item / per_tok), hm = (int)(item - (long)t * per_tok);
  const size_t at = (size_t)t * ldo + (size_t)hm * dv;
  if (tok_seq[t] < 0) {
    for (int c = threadIdx.x; c < dv; c += blockDim.x) {
      if (out_f32) ((float*)out)[at + c] = 0.f;
      else ((__nv_bfloat16*)out)[at + c] = __float2bfloat16_rn(0.f);
    }
    return;
  }
  const float* ml = ws_ml + (size_t)item * parts * 2;
  float M = -INFINITY;
  for (int s = 0; s < parts; ++s) M = fmaxf(M, ml[2 * s]);
  float part = 0.f;
  for (int s = threadIdx.x; s < parts; s += blockDim.x) {
    const float m = ml[2 * s];
    const float w = m == -INFINITY ? 0.f : exp2f(m - M);
    w_s[s] = w;
    part += w * ml[2 * s + 1];
  }
  float inv = 1.0f / block_sum(part, red);
  if (gate && gate_per <= 1) inv *= 1.0f / (1.0f + __expf(-gate[(size_t)t * ldg + hm / maps]));
  const float* o = ws_o + (size_t)item * parts * dv;
  for (int c = threadIdx.x; c < dv; c += blockDim.x) {
    float acc = 0.f;
    for (int s = 0; s < parts; ++s)
      if (w_s[s] != 0.f) acc = fmaf(w_s[s], o[(size_t)s * dv + c], acc);      // (a part that saw no key holds nothing)
    float res = acc * inv;
    if (gate && gate_per > 1) res *= 1.0f / (1.0f + __expf(-gate[(size_t)t * ldg + (size_t)hm * dv + c]));
    if (out_f32) ((float*)out)[at + c] = res;
    else ((__nv_bfloat16*)out)[at + c] = __float2bfloat16_rn(res);
  }
}

template <int NV, bool PROMPT>
int launch_maps_mma(const MapsArgs& a, dim3 grid, size_t smem, cudaStream_t stream) {
  static PerDevice<size_t> allowed;
  if (smem > 48 * 1024 && allowed.here() < smem) {
    if (cudaFuncSetAttribute(attention_maps_mma_kernel<NV, PROMPT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
      return LLMI_ERR_BAD_SIZE;
    allowed.here() = smem;
  }
  return launch_pdl(PDL_ATTENTION, attention_maps_mma_kernel<NV, PROMPT>, grid, dim3((PROMPT ? AM_PROMPT_WARPS : AM_WARPS) * 32), smem,
                    stream, a);
}

}  // namespace llmi

using namespace llmi;

LLMI_EXPORT int llmi_attention_maps_mma_supported(int dk, int dv, int group, int page_size) {
  const int nv = dv / 16;
  return dk > 0 && dv > 0 && dk % 16 == 0 && dv % 16 == 0 && dk <= 128 && dv <= 128 && (nv <= 4 || nv == 6 || nv == 8) &&
         group >= 1 && group <= 16 && page_size == AM_PAGE;
}

// floats of workspace of a step of single tokens
LLMI_EXPORT long llmi_attention_maps_mma_workspace(int n_tokens, int n_heads, int maps, int dv, int splits) {
  return (long)n_tokens * n_heads * maps * splits * (dv + 2);
}

// prompt != 0: n_blocks = an upper bound of the sum over sequences of ceil(tokens / 128).  prompt == 0: every sequence
// brings one token; `splits` cuts of `pages_per_split` pages over the visible positions.
LLMI_EXPORT int llmi_attention_maps_mma(const void* q, long ldq, void* out, long ldo, int out_f32, const void* k_cache,
                                        const void* v_cache, const int32_t* tok_seq, const int32_t* tok_pos,
                                        const int32_t* seq_pages, int pages_stride, const int32_t* seq_q_start,
                                        const int32_t* seq_kv_len, int n_tokens, int n_seqs, int n_heads, int n_kv_heads, int maps,
                                        int dk, int dv, float scale, const float* head_scale, int window, int chunk, int prompt,
                                        int n_blocks, int splits, int pages_per_split, float* workspace, long workspace_floats,
                                        int pool, const void* k_pool, const void* v_pool, const int32_t* pool_pages,
                                        int pool_pages_stride, const float* gate, long ldg, int gate_per, float softcap,
                                        cudaStream_t stream) {
  if (gate && gate_per != 1 && (gate_per != dv || maps != 1)) return LLMI_ERR_UNSUPPORTED;
  if (softcap < 0.f) return LLMI_ERR_BAD_SIZE;
  if (n_tokens <= 0 || n_seqs <= 0 || n_heads <= 0 || n_kv_heads <= 0 || maps <= 0 || n_heads % n_kv_heads) return LLMI_ERR_BAD_SIZE;
  if (!llmi_attention_maps_mma_supported(dk, dv, n_heads / n_kv_heads, AM_PAGE)) return LLMI_ERR_UNSUPPORTED;
  if (((uintptr_t)q & 15) || ((uintptr_t)k_cache & 15) || ((uintptr_t)v_cache & 15) || (ldq % 8) || ((uintptr_t)out & 7) || (ldo % 2))
    return LLMI_ERR_ALIGN;
  MapsArgs a;
  a.q = (const __nv_bfloat16*)q; a.ldq = ldq; a.out = out; a.ldo = ldo; a.out_f32 = out_f32;
  a.k_cache = (const __nv_bfloat16*)k_cache; a.v_cache = (const __nv_bfloat16*)v_cache;
  a.tok_seq = tok_seq; a.tok_pos = tok_pos; a.seq_pages = seq_pages; a.pages_stride = pages_stride;
  a.seq_q_start = seq_q_start; a.seq_kv_len = seq_kv_len;
  a.n_seqs = n_seqs; a.H = n_heads; a.G = n_kv_heads; a.maps = maps; a.dk = dk;
  a.scale_log2 = scale * 1.4426950408889634f; a.head_scale = head_scale; a.window = window; a.chunk = chunk;
  a.splits = splits; a.pages_per_split = pages_per_split; a.ws_o = nullptr; a.ws_ml = nullptr;
  if (pool < 0 || (pool > 0 && (!k_pool || !v_pool || !pool_pages || window <= 0 || ((uintptr_t)k_pool & 15) || ((uintptr_t)v_pool & 15))))
    return LLMI_ERR_BAD_SIZE;
  a.pool = pool; a.k_pool = (const __nv_bfloat16*)k_pool; a.v_pool = (const __nv_bfloat16*)v_pool;
  a.pool_pages = pool_pages; a.pool_pages_stride = pool_pages_stride; a.gate = gate; a.ldg = ldg;
  a.gate_per = gate_per; a.softcap_log2 = softcap * 1.4426950408889634f;
  const int rows = prompt ? AM_PROMPT_ROWS : 16;
  const int nbuf = prompt ? 2 : AM_TOKEN_BUFFERS;
  const size_t smem = ((size_t)(rows + nbuf * AM_PAGE) * (dk + AM_PAD) + (size_t)nbuf * AM_PAGE * (dv + AM_PAD)) * 2;
  dim3 grid;
  if (prompt) {
    if (n_blocks <= 0 || n_heads * maps > 65535) return LLMI_ERR_BAD_SIZE;
    grid = dim3(n_blocks, n_heads * maps);
  } else {
    if (splits < 1 || pages_per_split < 1 || splits > AM_MAX_PARTS || n_kv_heads * maps > 65535 || splits > 65535) return LLMI_ERR_BAD_SIZE;
    const long need = llmi_attention_maps_mma_workspace(n_tokens, n_heads, maps, dv, splits);
    if (!workspace || workspace_floats < need) return LLMI_ERR_BAD_SIZE;
    a.ws_o = workspace;
    a.ws_ml = workspace + (size_t)n_tokens * n_heads * maps * splits * dv;
    grid = dim3(n_seqs, n_kv_heads * maps, splits);
  }
  int rc;
#define LLMI_CASE(NVV) \
  case NVV: rc = prompt ? launch_maps_mma<NVV, true>(a, grid, smem, stream) : launch_maps_mma<NVV, false>(a, grid, smem, stream); break
  switch (dv / 16) {
    LLMI_CASE(1); LLMI_CASE(2); LLMI_CASE(3); LLMI_CASE(4); LLMI_CASE(6); LLMI_CASE(8);
    default: return LLMI_ERR_UNSUPPORTED;
  }
#undef LLMI_CASE
  if (rc != LLMI_OK || prompt || splits == 1) return rc;
  const long items = (long)n_tokens * n_heads * maps;
  if (items > 0x7fffffffL) return LLMI_ERR_BAD_SIZE;
  return launch_pdl(PDL_SMALL, attention_maps_join_kernel, dim3((unsigned)items), dim3(128), 0, stream, (const float*)a.ws_o,
                    (const float*)a.ws_ml, out, ldo, out_f32, tok_seq, n_heads * maps, dv, splits, gate, ldg, maps, gate_per);
}
