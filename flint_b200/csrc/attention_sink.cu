// Paged attention in its general form: keys and values of different sizes, a sliding window that keeps a
// request's first tokens, and a learned sink logit per query head in the softmax's denominator.
//
// A query row t at position p of request slot[t] sees key j of its request if j <= p and (p - j < window or
// j < keep_first); window 0: every j <= p.  Instead of a window a layer may cut the sequence into runs of `run`
// positions counted from 0: then j is seen if j <= p and floor(j / run) = floor(p / run).  The seen keys are numbered without gaps: first the kept ones below
// the window's start (positions 0 .. min(keep_first, lo) - 1, lo = max(0, p + 1 - window)), then lo .. p; a split
// of the key range is a run of these numbers.  Kept tokens keep their positions: they were rotated where they
// stand, and nothing is rotated again.  With a sink s_h the weights are e^(score_j - M) / (sum_j e^(score_j - M)
// + e^(s_h - M)): the sink takes part in the maximum and the sum and has no value.  Scores, maxima, sums and the
// output are float32 (online softmax over blocks of 32 keys).
//
// flint_qkv_write makes q and the cache rows from the projection: it adds up the partial sums and the bias,
// rotates the leading `rot` dims of every query and key head by the token's position, optionally leaves the
// values as projected for later layers (v_keep) or blends them with an earlier layer's (v = (1 - a) v + a v_from),
// and writes keys [page, kv head, P, hd] and values [page, kv head, P, vd] into the token's page.
//
// Work of flint_sink_attention is split as (row, kv head, chunk of up to 4 query heads, split): one warp each;
// a lane owns a key in the score phase and value dims lane, lane + 32, ... in the value phase.  With several
// splits a second kernel merges (max, sum, unnormalised output) records in a fixed order and adds the sink.
// Head sizes up to 256; rows of whole 16-byte units are read in such units, others element by element.
//
// The reference's attention has the causal and window mask only (crates/thuban_kernel/wgsl/attn.wgsl:78-90).
#include <math.h>
#include <stdarg.h>
#include "common.cuh"

using namespace flint;

namespace {

constexpr int GC = 4;          // query heads per warp
constexpr int WARPS = 4;
constexpr int MAX_DPL = 8;     // value dims per lane: vd <= 256

template <typename TC> struct Vec8;
template <> struct Vec8<float> {
  static __device__ __forceinline__ void load(const float* p, float* f) {
    const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
    f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
  }
};
template <> struct Vec8<__nv_bfloat16> {
  static __device__ __forceinline__ void load(const __nv_bfloat16* p, float* f) {
    const uint4 a = *reinterpret_cast<const uint4*>(p);
    const uint32_t w[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      f[2 * i] = __uint_as_float(w[i] << 16);
      f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
  }
};

// ------------------------------------------------------------------------------------------- q and the cache rows
template <typename TQ, typename TC>
__global__ void qkv_write_kernel(const float* __restrict__ qkv, int n_partials, long long partial_stride,
                                 const float* __restrict__ bias, const int* __restrict__ pos, const int* __restrict__ slot,
                                 const float* __restrict__ cos_t, const float* __restrict__ sin_t, int rot, int interleaved,
                                 TQ* __restrict__ q_out, TC* __restrict__ k_cache, TC* __restrict__ v_cache,
                                 const int* __restrict__ block_table, int max_pages, int page_size, int nq, int nkv,
                                 int hd, int vd, float* __restrict__ v_keep, const float* __restrict__ v_from, float blend,
                                 int* __restrict__ status) {
  pdl_launch();
  pdl_wait();
  const int t = blockIdx.x;
  const int p = pos[t];
  const int lp = p / page_size;
  const int page = lp < max_pages ? block_table[(size_t)slot[t] * max_pages + lp] : -1;
  if (page < 0 && threadIdx.x == 0) atomicExch(status, 1);
  const int qk_w = (nq + nkv) * hd, W = qk_w + nkv * vd, half = rot / 2;
  const float* row = qkv + (size_t)t * W;
  auto value = [&](int e) {
    float x = 0.f;
    for (int z = 0; z < n_partials; ++z) x += row[(size_t)z * partial_stride + e];
    return bias ? x + bias[e] : x;
  };
  for (int e = threadIdx.x; e < W; e += blockDim.x) {
    float x = value(e);
    if (e < qk_w) {
      const int head = e / hd, d = e % hd;
      if (d < rot) {
        int i, partner;
        bool first;
        if (interleaved) { i = d >> 1; first = !(d & 1); partner = first ? e + 1 : e - 1; }
        else { i = d < half ? d : d - half; first = d < half; partner = first ? e + half : e - half; }
        const float y = value(partner);
        const float c = cos_t[(size_t)p * half + i], s = sin_t[(size_t)p * half + i];
        x = first ? x * c - y * s : x * c + y * s;
      }
      if (head < nq) {
        q_out[(size_t)t * nq * hd + e] = from_f32<TQ>(x);
      } else if (page >= 0) {
        k_cache[(((size_t)page * nkv + (head - nq)) * page_size + p % page_size) * hd + d] = from_f32<TC>(x);
      }
    } else {
      const int ev = e - qk_w, kvh = ev / vd, d = ev % vd;
      if (v_keep) v_keep[(size_t)t * nkv * vd + ev] = x;
      if (v_from) x = (1.0f - blend) * x + blend * v_from[(size_t)t * nkv * vd + ev];
      if (page >= 0) v_cache[(((size_t)page * nkv + kvh) * page_size + p % page_size) * vd + d] = from_f32<TC>(x);
    }
  }
}

// ------------------------------------------------------------------------------------------- means of blocks of keys and values
// A row whose position p ends a block of `pool` positions (p + 1 a multiple of pool) writes the block's mean key and
// mean value, taken over the cache rows as they stand (so after norm and rotation, and in the cache's precision), in
// float32 and in the order of the positions, into row b = (p + 1) / pool - 1 of the request's block means: slot
// b % pool_slots of the request's page b / pool_slots, pool_slots = ceil(page_size / pool) means a page (that page
// is one the request already holds: b / pool_slots <= (b pool + pool - 1) / page_size).  Whatever the cut of a
// prompt, a block is written once, by the step that brings its last position, after that step's cache rows.
template <typename TC>
__global__ void pool_write_kernel(const TC* __restrict__ k_cache, const TC* __restrict__ v_cache, TC* __restrict__ pool_k,
                                  TC* __restrict__ pool_v, const int* __restrict__ block_table, int max_pages,
                                  int page_size, const int* __restrict__ pos, const int* __restrict__ slot, int nkv, int hd,
                                  int vd, int pool, int pool_slots, int* __restrict__ status) {
  pdl_launch();
  pdl_wait();
  const int t = blockIdx.x, kvh = blockIdx.y, p = pos[t];
  if ((p + 1) % pool) return;
  const int b = (p + 1) / pool - 1, j0 = b * pool;
  const int* bt = block_table + (size_t)slot[t] * max_pages;
  const int home = b / pool_slots < max_pages ? bt[b / pool_slots] : -1;
  if (home < 0) {
    if (threadIdx.x == 0) atomicExch(status, 1);
    return;
  }
  const size_t dst = ((size_t)home * nkv + kvh) * pool_slots + b % pool_slots;
  const float share = 1.0f / (float)pool;
  for (int d = threadIdx.x; d < hd + vd; d += blockDim.x) {
    float sum = 0.f;
    for (int j = j0; j <= p; ++j) {
      const int page = bt[j / page_size];
      if (page < 0) { atomicExch(status, 1); continue; }
      const size_t at = ((size_t)page * nkv + kvh) * page_size + j % page_size;
      sum += d < hd ? to_f32(k_cache[at * hd + d]) : to_f32(v_cache[at * vd + (d - hd)]);
    }
    if (d < hd) pool_k[dst * hd + d] = from_f32<TC>(sum * share);
    else pool_v[dst * vd + (d - hd)] = from_f32<TC>(sum * share);
  }
}

// Weights without a softmax (see the attention kernel): on, the cap of the scores (0: none), per query head the
// distance penalty's two numbers and the bias (null: none).
struct SigmoidWeights {
  int on;
  float cap;
  const float* r1;
  const float* r2;
  const float* bias;
};

// ------------------------------------------------------------------------------------------- attention
// DPL: value dims a lane holds (vd <= 32 DPL); the narrow forms keep fewer registers, so more blocks fit an SM and
// hide each other's waits for their key rows.
template <typename TQ, typename TC, typename TO, int DPL>
__global__ void __launch_bounds__(WARPS * 32, DPL <= 4 ? 6 : 3)
sink_attention_kernel(const TQ* __restrict__ q, const TC* __restrict__ k_cache, const TC* __restrict__ v_cache,
                      const int* __restrict__ block_table, int max_pages, int page_size, const int* __restrict__ pos,
                      const int* __restrict__ slot, TO* __restrict__ out, float* __restrict__ scratch, int T, int nq,
                      int nkv, int hd, int vd, int window, int keep_first, int run, const float* __restrict__ sinks, float scale,
                      int split_keys, int n_splits, int g_chunks, const int* __restrict__ row_list,
                      const TC* __restrict__ pool_k, const TC* __restrict__ pool_v, int pool, int pool_slots, SigmoidWeights sw) {
  extern __shared__ float smem[];  // per warp: GC * hd floats of q
  pdl_launch();
  pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long item = (long long)blockIdx.x * WARPS + warp;
  if (item >= (long long)T * nkv * g_chunks * n_splits) return;
  const int split = (int)(item % n_splits);
  long long rest = item / n_splits;
  const int gchunk = (int)(rest % g_chunks);
  rest /= g_chunks;
  const int kvh = (int)(rest % nkv);
  const int ti = (int)(rest / nkv);                  // index into the rows this launch covers
  const int t = row_list ? row_list[ti] : ti;        // row of the batch
  const int G = nq / nkv, g0 = gchunk * GC, ng = min(GC, G - g0), h0 = kvh * G + g0;
  const int p = pos[t];
  // the first key of the stretch that ends at p: the window's start, or the start of p's run of `run` positions
  const int lo = run > 0 ? (p / run) * run : (window > 0 ? max(0, p + 1 - window) : 0);
  // keys below the window's start: the kept first ones, or one mean key per block of `pool` positions that lies
  // wholly below it (block b, positions b pool .. b pool + pool - 1, if b pool + pool - 1 <= p - window)
  const int n_first = pool > 0 ? max(0, (p - window + 1) / pool) : min(keep_first, lo);
  const int total = n_first + (p + 1 - lo);             // seen keys, numbered 0 .. total - 1
  const int u_lo = split * split_keys, u_hi = min(total, u_lo + split_keys);
  const int* bt = block_table + (size_t)slot[t] * max_pages;

  float* qs = smem + warp * GC * hd;
  for (int i = lane; i < ng * hd; i += 32) qs[i] = to_f32(q[((size_t)t * nq + h0) * hd + i]) * scale;
  __syncwarp();

  const bool k_vec = (hd % 8) == 0;
  const int dpl = (vd + 31) / 32;
  float m[GC], l[GC], acc[GC][DPL];
#pragma unroll
  for (int g = 0; g < GC; ++g) {
    m[g] = -INFINITY;
    l[g] = 0.f;
#pragma unroll
    for (int i = 0; i < DPL; ++i) acc[g][i] = 0.f;
  }

  for (int u0 = u_lo; u0 < u_hi; u0 += 32) {
    const int u = u0 + lane;
    long long row = -1;   // index of the key's row in [page, kv_head, P] units; -2 - (its row among the block means)
    int dist = 0;         // how far behind the query the key lies
    if (u < u_hi) {
      if (pool > 0 && u < n_first) {
        const int page = bt[u / pool_slots];
        if (page >= 0) row = -2 - (((long long)page * nkv + kvh) * pool_slots + (u % pool_slots));
      } else {
        const int j = u < n_first ? u : lo + (u - n_first);
        const int page = bt[j / page_size];
        if (page >= 0) row = ((long long)page * nkv + kvh) * page_size + (j % page_size);
        dist = p - j;
      }
    }
    const bool have = row != -1;
    float s[GC];
#pragma unroll
    for (int g = 0; g < GC; ++g) s[g] = 0.f;
    if (have) {
      const TC* kr = row >= 0 ? k_cache + row * hd : pool_k + (-2 - row) * hd;
      if (k_vec) {
#pragma unroll 2
        for (int d = 0; d < hd; d += 8) {
          float kf[8];
          Vec8<TC>::load(kr + d, kf);
#pragma unroll
          for (int g = 0; g < GC; ++g)
            if (g < ng) {
#pragma unroll
              for (int e = 0; e < 8; ++e) s[g] = fmaf(qs[g * hd + d + e], kf[e], s[g]);
            }
        }
      } else {
        for (int d = 0; d < hd; ++d) {
          const float kf = to_f32(kr[d]);
#pragma unroll
          for (int g = 0; g < GC; ++g)
            if (g < ng) s[g] = fmaf(qs[g * hd + d], kf, s[g]);
        }
      }
    }
    float pr[GC];
    if (sw.on) {
      // no softmax: a key's weight is sigmoid(cap tanh(score / cap) - r1 ln(1 + r2 distance) + bias), not normalised
#pragma unroll
      for (int g = 0; g < GC; ++g) {
        float z = s[g];
        if (sw.cap > 0.f) z = sw.cap * tanhf(z / sw.cap);
        if (g < ng) {
          if (sw.r1) z -= sw.r1[h0 + g] * logf(1.0f + sw.r2[h0 + g] * (float)dist);
          if (sw.bias) z += sw.bias[h0 + g];
        }
        pr[g] = have ? 1.0f / (1.0f + expf(-z)) : 0.f;
      }
    } else {
#pragma unroll
      for (int g = 0; g < GC; ++g) {
        const float sg = have ? s[g] : -INFINITY;
        const float m_new = fmaxf(m[g], warp_max(sg));
        const bool any = m_new > -INFINITY;
        const float alpha = any ? expf(m[g] - m_new) : 1.f;
        pr[g] = (any && have) ? expf(sg - m_new) : 0.f;
        l[g] = l[g] * alpha + warp_sum(pr[g]);
        m[g] = m_new;
#pragma unroll
        for (int i = 0; i < DPL; ++i) acc[g][i] *= alpha;
      }
    }
    const int nk = min(32, u_hi - u0);
    constexpr int VU = 4;      // value rows in flight per lane
    for (int jj0 = 0; jj0 < nk; jj0 += VU) {
      float vv[VU][DPL];
#pragma unroll
      for (int u = 0; u < VU; ++u) {
        const long long vrow = __shfl_sync(0xffffffffu, row, (jj0 + u) & 31);
        const bool ok = jj0 + u < nk && vrow != -1;
        const TC* vr = !ok ? v_cache : (vrow >= 0 ? v_cache + vrow * vd : pool_v + (-2 - vrow) * vd);
#pragma unroll
        for (int i = 0; i < DPL; ++i) {
          const int d = lane + 32 * i;
          vv[u][i] = (ok && i < dpl && d < vd) ? to_f32(vr[d]) : 0.f;
        }
      }
#pragma unroll
      for (int u = 0; u < VU; ++u) {
        float pj[GC];
#pragma unroll
        for (int g = 0; g < GC; ++g) pj[g] = __shfl_sync(0xffffffffu, pr[g], (jj0 + u) & 31);
        if (jj0 + u >= nk) continue;          // the same for every lane
#pragma unroll
        for (int i = 0; i < DPL; ++i)
          if (i < dpl) {
#pragma unroll
            for (int g = 0; g < GC; ++g) acc[g][i] = fmaf(pj[g], vv[u][i], acc[g][i]);
          }
      }
    }
  }

  if (n_splits == 1) {
#pragma unroll
    for (int g = 0; g < GC; ++g)
      if (g < ng) {
        float scale_o = 1.f, sum = l[g];
        if (sw.on) sum = 1.f;          // the weights are used as they are
        else if (sinks) {      // the sink joins the maximum and the sum
          const float sk = sinks[h0 + g], m_all = fmaxf(m[g], sk);
          scale_o = m[g] > -INFINITY ? expf(m[g] - m_all) : 0.f;
          sum = l[g] * scale_o + expf(sk - m_all);
        }
        const float inv = sum > 0.f ? scale_o / sum : 0.f;
#pragma unroll
        for (int i = 0; i < DPL; ++i) {
          const int d = lane + 32 * i;
          if (i < dpl && d < vd) out[((size_t)t * nq + h0 + g) * vd + d] = from_f32<TO>(acc[g][i] * inv);
        }
      }
  } else {
    // scratch [T, nq, n_splits, vd + 2]: unnormalised output, then max, then sum
#pragma unroll
    for (int g = 0; g < GC; ++g)
      if (g < ng) {
        float* dst = scratch + (((size_t)ti * nq + h0 + g) * n_splits + split) * (vd + 2);
#pragma unroll
        for (int i = 0; i < DPL; ++i) {
          const int d = lane + 32 * i;
          if (i < dpl && d < vd) dst[d] = acc[g][i];
        }
        if (lane == 0) {
          dst[vd] = m[g];
          dst[vd + 1] = l[g];
        }
      }
  }
}

// Merge the splits of one (row, head) and add the sink: out = sum_s e^(m_s - M) o_s / (sum_s e^(m_s - M) l_s + e^(sink - M)).
template <typename TO>
__global__ void sink_combine_kernel(const float* __restrict__ scratch, TO* __restrict__ out, int vd, int n_splits, int nq,
                                    const float* __restrict__ sinks, const int* __restrict__ row_list, int plain_sum) {
  pdl_launch();
  pdl_wait();
  const size_t rh = blockIdx.x;   // (index of the row in this launch) * nq + head
  const size_t out_rh = row_list ? (size_t)row_list[rh / nq] * nq + rh % nq : rh;
  const float* base = scratch + rh * n_splits * (vd + 2);
  if (plain_sum) {                // weights that are not normalised: the splits' sums add up, in a fixed order
    for (int d = threadIdx.x; d < vd; d += blockDim.x) {
      float o = 0.f;
      for (int s = 0; s < n_splits; ++s) o += base[(size_t)s * (vd + 2) + d];
      out[out_rh * vd + d] = from_f32<TO>(o);
    }
    return;
  }
  const float sk = sinks ? sinks[rh % nq] : -INFINITY;
  float M = sk;
  for (int s = 0; s < n_splits; ++s) M = fmaxf(M, base[(size_t)s * (vd + 2) + vd]);
  float L = sinks ? expf(sk - M) : 0.f;
  for (int s = 0; s < n_splits; ++s) {           // fixed order, the same in every thread
    const float ms = base[(size_t)s * (vd + 2) + vd];
    if (ms > -INFINITY) L += expf(ms - M) * base[(size_t)s * (vd + 2) + vd + 1];
  }
  const float inv = L > 0.f ? 1.0f / L : 0.f;
  for (int d = threadIdx.x; d < vd; d += blockDim.x) {
    float o = 0.f;
    for (int s = 0; s < n_splits; ++s) {
      const float ms = base[(size_t)s * (vd + 2) + vd];
      if (ms > -INFINITY) o += expf(ms - M) * base[(size_t)s * (vd + 2) + d];
    }
    out[out_rh * vd + d] = from_f32<TO>(o * inv);
  }
}


// ------------------------------------------------------------------------------------------- long portions on the tensor cores
// Tiles of up to 64 consecutive rows of one request (bfloat16, head sizes in multiples of 16 up to 128): a block of four
// warps takes a tile and a query head, a warp 16 rows.  The keys the tile's rows see between them (the kept first ones,
// then from the first row's window start to the last row's position) are walked in tiles of 64: keys and values come
// into shared memory by asynchronous 16-byte copies (rows padded by 16 bytes, so ldmatrix meets no bank twice),
// S = Q K^T by mma.sync m16n8k16 with Q's fragments in registers, the mask (not later; near, or kept) and the online
// softmax in float32 on the accumulator fragment, P as bfloat16 the A operand of O += P V with V through ldmatrix.trans.
// The sink joins maximum and sum at the end.
constexpr int MQ = 64, MK = 64;      // query rows a block, keys a tile
static_assert(MK * 2 == 128, "two of the block's 128 threads fetch a key");

__device__ __forceinline__ void ldsm4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldsm4t(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void mma16816(float* d, const uint32_t* a, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
               "{%0, %1, %2, %3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void copy16(void* dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ float tanh_fast(float x) {
  float y;
  asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&v);
}

// HDS: most k steps of 16 query/key dims; VDT: most tiles of 8 value dims
template <int HDS, int VDT>
__global__ void __launch_bounds__(128)
sink_attention_mma_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k_cache,
                          const __nv_bfloat16* __restrict__ v_cache, const int* __restrict__ block_table, int max_pages,
                          int page_size, const int* __restrict__ tiles, __nv_bfloat16* __restrict__ out, int nq, int nkv, int hd,
                          int vd, int window, int keep_first, int run, const float* __restrict__ sinks, float scale,
                          const __nv_bfloat16* __restrict__ pool_k, const __nv_bfloat16* __restrict__ pool_v, int pool,
                          int pool_slots, SigmoidWeights sw) {
  extern __shared__ __align__(16) unsigned char sm_raw[];
  const int ldk = hd + 8, ldv = vd + 8;
  // two stages, each keys [MK][ldk], values [MK][ldv] and the keys' positions [MK] (or -1); the first stage's keys
  // first hold the query tile
  const int stage_bytes = MK * (ldk + ldv) * 2 + MK * (int)sizeof(int);
  pdl_launch();
  pdl_wait();
  const int tile = blockIdx.x / nq, h = blockIdx.x % nq, kvh = h / (nq / nkv);
  const int row0 = tiles[4 * tile], n_rows = tiles[4 * tile + 1], slot = tiles[4 * tile + 2], p0 = tiles[4 * tile + 3];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, tq = lane & 3;
  const int hd16 = hd / 16, vdt = vd / 8, chunks_k = hd / 8, chunks_v = vd / 8;
  const int lm = lane >> 3, lr = lane & 7;                             // ldmatrix: this lane addresses row lr of matrix lm

  {
    __nv_bfloat16* q_s = reinterpret_cast<__nv_bfloat16*>(sm_raw);
    for (int i = tid; i < MQ * chunks_k; i += 128) {
      const int r = i / chunks_k, c = i % chunks_k;
      uint4 val = make_uint4(0u, 0u, 0u, 0u);
      if (r < n_rows) val = *reinterpret_cast<const uint4*>(q + ((size_t)(row0 + r) * nq + h) * hd + c * 8);
      *reinterpret_cast<uint4*>(q_s + r * ldk + c * 8) = val;
    }
    __syncthreads();
  }
  uint32_t qf[HDS][4];
#pragma unroll
  for (int ks = 0; ks < HDS; ++ks)
    if (ks < hd16) {
      const __nv_bfloat16* src = reinterpret_cast<__nv_bfloat16*>(sm_raw) + (warp * 16 + (lm & 1) * 8 + lr) * ldk + ks * 16 + (lm >> 1) * 8;
      ldsm4((uint32_t)__cvta_generic_to_shared(src), qf[ks][0], qf[ks][1], qf[ks][2], qf[ks][3]);
    }
  __syncthreads();          // the query tile's place is free for keys

  const int p_last = p0 + n_rows - 1;
  const int lo_first = run > 0 ? (p0 / run) * run : (window > 0 ? max(0, p0 + 1 - window) : 0);
  const bool gap = (window > 0 || run > 0) && lo_first > keep_first;  // kept keys and window do not touch
  // with block means: first the means the tile's last row sees (a key "position" -2 - b stands for block b), then
  // the positions from the first row's window start on
  const int n_first = pool > 0 ? max(0, (p_last - window + 1) / pool) : (gap ? keep_first : 0);
  const int base = pool > 0 ? lo_first : (gap ? lo_first : 0);
  const int total = n_first + (p_last + 1 - base);
  const int* bt = block_table + (size_t)slot * max_pages;
  const int r_lo = warp * 16 + g;                                      // this thread's two rows: r_lo and r_lo + 8
  const int p_row[2] = {p0 + r_lo, p0 + r_lo + 8};
  const bool row_ok[2] = {r_lo < n_rows, r_lo + 8 < n_rows};
  float m_r[2] = {-INFINITY, -INFINITY}, l_r[2] = {0.f, 0.f};
  float o[VDT][4];
#pragma unroll
  for (int nt = 0; nt < VDT; ++nt)
#pragma unroll
    for (int e = 0; e < 4; ++e) o[nt][e] = 0.f;

  // the copies of one tile of keys and values into a stage; the next tile's are on their way while this one is worked
  auto fetch = [&](int u0, int stage) {
    __nv_bfloat16* k_d = reinterpret_cast<__nv_bfloat16*>(sm_raw + (size_t)stage * stage_bytes);
    __nv_bfloat16* v_d = k_d + MK * ldk;
    int* pos_d = reinterpret_cast<int*>(v_d + MK * ldv);
    auto key_at = [&](int r) {
      const int u = u0 + r;
      return u < total ? (u < n_first ? (pool > 0 ? -2 - u : u) : base + (u - n_first)) : -1;
    };
    // two threads a key: the key's position and page are worked out once, then the row's 16-byte pieces alternate
    const int r = tid >> 1, half = tid & 1, j = key_at(r);
    if (half == 0) pos_d[r] = j;
    const int blk = -2 - j;                    // the block whose means stand at this place, if j <= -2
    const int page = j >= 0 ? bt[j / page_size] : (j <= -2 ? bt[blk / pool_slots] : -1);
    __nv_bfloat16* kd = k_d + r * ldk;
    __nv_bfloat16* vd_ = v_d + r * ldv;
    if (page >= 0) {
      const size_t at = j >= 0 ? ((size_t)page * nkv + kvh) * page_size + j % page_size
                               : ((size_t)page * nkv + kvh) * pool_slots + blk % pool_slots;
      const __nv_bfloat16* ks = (j >= 0 ? k_cache : pool_k) + at * hd;
      const __nv_bfloat16* vs = (j >= 0 ? v_cache : pool_v) + at * vd;
      for (int c = half; c < chunks_k; c += 2) copy16(kd + c * 8, ks + c * 8);
      for (int c = half; c < chunks_v; c += 2) copy16(vd_ + c * 8, vs + c * 8);
    } else {
      for (int c = half; c < chunks_k; c += 2) *reinterpret_cast<uint4*>(kd + c * 8) = make_uint4(0u, 0u, 0u, 0u);
      for (int c = half; c < chunks_v; c += 2) *reinterpret_cast<uint4*>(vd_ + c * 8) = make_uint4(0u, 0u, 0u, 0u);
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  fetch(0, 0);
  int stage = 0;
  for (int u0 = 0; u0 < total; u0 += MK, stage ^= 1) {
    if (u0 + MK < total) {
      fetch(u0 + MK, stage ^ 1);
      asm volatile("cp.async.wait_group 1;" ::: "memory");
    } else {
      asm volatile("cp.async.wait_group 0;" ::: "memory");
    }
    __syncthreads();
    const __nv_bfloat16* k_s = reinterpret_cast<const __nv_bfloat16*>(sm_raw + (size_t)stage * stage_bytes);
    const __nv_bfloat16* v_s = k_s + MK * ldk;
    const int* kpos = reinterpret_cast<const int*>(v_s + MK * ldv);

    float s[MK / 8][4];
#pragma unroll
    for (int nt = 0; nt < MK / 8; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) s[nt][e] = 0.f;
#pragma unroll
    for (int ks = 0; ks < HDS; ++ks)
      if (ks < hd16) {
#pragma unroll
        for (int np = 0; np < MK / 16; ++np) {
          uint32_t b0, b1, b2, b3;
          const __nv_bfloat16* src = k_s + (np * 16 + (lm >> 1) * 8 + lr) * ldk + ks * 16 + (lm & 1) * 8;
          ldsm4((uint32_t)__cvta_generic_to_shared(src), b0, b1, b2, b3);
          mma16816(s[2 * np], qf[ks], b0, b1);
          mma16816(s[2 * np + 1], qf[ks], b2, b3);
        }
      }
    // mask, scale, and this tile's maxima of the thread's two rows.  Most tiles lie behind every row of the tile and
    // inside every row's window: they need no mask
    float mx[2] = {-INFINITY, -INFINITY};
    const bool interior = !sw.on &&
        ((kpos[0] >= 0 && kpos[MK - 1] >= 0 && kpos[MK - 1] <= p0 && (window == 0 || p_last - kpos[0] < window) &&
          (run == 0 || kpos[0] >= (p_last / run) * run)) ||
         (kpos[MK - 1] <= -2 && (-1 - kpos[MK - 1]) * pool <= p0 - window + 1));     // or means that every row sees
    if (sw.on) {
      // no softmax: a key's weight is sigmoid(cap tanh(score / cap) - r1 ln(1 + r2 distance) + bias), not normalised
      const float r1 = sw.r1 ? sw.r1[h] : 0.f, r2 = sw.r2 ? sw.r2[h] : 0.f, wb = sw.bias ? sw.bias[h] : 0.f;
      const float inv_cap = sw.cap > 0.f ? 1.0f / sw.cap : 0.f;
#pragma unroll
      for (int nt = 0; nt < MK / 8; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int j = kpos[nt * 8 + 2 * tq + (e & 1)], rs = e >> 1, p = p_row[rs];
          const bool ok = j >= 0 && row_ok[rs] && j <= p && (window == 0 || p - j < window);
          // bfloat16 follows: the single-instruction forms of tanh and the logarithm will do, and
          // sigmoid(x) = (1 + tanh(x / 2)) / 2
          float z = s[nt][e] * scale;
          if (sw.cap > 0.f) z = sw.cap * tanh_fast(z * inv_cap);
          if (sw.r1) z -= r1 * __logf(fmaf(r2, (float)(p - j), 1.0f));
          s[nt][e] = ok ? fmaf(0.5f, tanh_fast(0.5f * (z + wb)), 0.5f) : 0.f;
        }
    } else if (interior) {
#pragma unroll
      for (int nt = 0; nt < MK / 8; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          s[nt][e] *= scale;
          mx[e >> 1] = fmaxf(mx[e >> 1], s[nt][e]);
        }
    } else {
#pragma unroll
      for (int nt = 0; nt < MK / 8; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int j = kpos[nt * 8 + 2 * tq + (e & 1)], rs = e >> 1, p = p_row[rs];
          const bool ok = j <= -2 ? row_ok[rs] && (-1 - j) * pool <= p - window + 1
                                  : j >= 0 && row_ok[rs] && j <= p && (window == 0 || p - j < window || j < keep_first) &&
                                        (run == 0 || j >= (p / run) * run);
          s[nt][e] = ok ? s[nt][e] * scale : -INFINITY;
          mx[rs] = fmaxf(mx[rs], s[nt][e]);
        }
    }
    float alpha[2] = {1.f, 1.f};
    if (!sw.on) {
#pragma unroll
    for (int rs = 0; rs < 2; ++rs) {
      mx[rs] = fmaxf(mx[rs], __shfl_xor_sync(0xffffffffu, mx[rs], 1));
      mx[rs] = fmaxf(mx[rs], __shfl_xor_sync(0xffffffffu, mx[rs], 2));
      const float m_new = fmaxf(m_r[rs], mx[rs]);
      alpha[rs] = m_new > -INFINITY ? __expf(m_r[rs] - m_new) : 1.f;    // 0 while m_r is still -inf
      m_r[rs] = m_new;
    }
    float sum[2] = {0.f, 0.f};
#pragma unroll
    for (int nt = 0; nt < MK / 8; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int rs = e >> 1;
        const float pv = s[nt][e] > -INFINITY ? __expf(s[nt][e] - m_r[rs]) : 0.f;     // bfloat16 follows: the fast form will do
        s[nt][e] = pv;
        sum[rs] += pv;
      }
#pragma unroll
    for (int rs = 0; rs < 2; ++rs) {
      sum[rs] += __shfl_xor_sync(0xffffffffu, sum[rs], 1);
      sum[rs] += __shfl_xor_sync(0xffffffffu, sum[rs], 2);
      l_r[rs] = l_r[rs] * alpha[rs] + sum[rs];
    }
#pragma unroll
    for (int nt = 0; nt < VDT; ++nt) {
      o[nt][0] *= alpha[0]; o[nt][1] *= alpha[0];
      o[nt][2] *= alpha[1]; o[nt][3] *= alpha[1];
    }
    }
#pragma unroll
    for (int kk = 0; kk < MK / 16; ++kk) {
      const uint32_t a[4] = {pack_bf16(s[2 * kk][0], s[2 * kk][1]), pack_bf16(s[2 * kk][2], s[2 * kk][3]),
                             pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]), pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3])};
#pragma unroll
      for (int vp = 0; vp < VDT / 2; ++vp)
        if (2 * vp < vdt) {
          uint32_t b0, b1, b2, b3;
          const __nv_bfloat16* src = v_s + (kk * 16 + (lm & 1) * 8 + lr) * ldv + vp * 16 + (lm >> 1) * 8;
          ldsm4t((uint32_t)__cvta_generic_to_shared(src), b0, b1, b2, b3);
          mma16816(o[2 * vp], a, b0, b1);
          mma16816(o[2 * vp + 1], a, b2, b3);
        }
    }
    __syncthreads();        // this stage is refilled in the next round
  }

#pragma unroll
  for (int rs = 0; rs < 2; ++rs) {
    if (!row_ok[rs]) continue;
    float so = 1.f, sum = l_r[rs];
    if (sw.on) sum = 1.f;
    else if (sinks) {
      const float sk = sinks[h], m_all = fmaxf(m_r[rs], sk);
      so = m_r[rs] > -INFINITY ? expf(m_r[rs] - m_all) : 0.f;
      sum = l_r[rs] * so + expf(sk - m_all);
    }
    const float inv = sum > 0.f ? so / sum : 0.f;
    __nv_bfloat16* dst = out + ((size_t)(row0 + r_lo + 8 * rs) * nq + h) * vd + 2 * tq;
#pragma unroll
    for (int nt = 0; nt < VDT; ++nt)
      if (nt < vdt)
        *reinterpret_cast<uint32_t*>(dst + nt * 8) = pack_bf16(o[nt][2 * rs] * inv, o[nt][2 * rs + 1] * inv);
  }
}

}  // namespace

extern "C" int flint_qkv_write(const float* qkv, int n_partials, long long partial_stride, const float* bias,
                               const int* pos, const int* slot, const float* cos_t, const float* sin_t, int rot,
                               int interleaved, void* q_out, int q_dtype, void* k_cache, void* v_cache, int cache_dtype,
                               const int* block_table, int max_pages, int page_size, int T, int nq, int nkv, int hd,
                               int vd, float* v_keep, const float* v_from, float blend, int* status,
                               cudaStream_t stream) {
  if (T <= 0) return 0;
  if (n_partials < 1) return fail("qkv_write: needs at least one partial");
  if (rot < 0 || rot > hd || (rot & 1)) return fail("qkv_write: %d rotating dims do not fit head size %d", rot, hd);
  if (page_size <= 0 || nq < 1 || nkv < 1 || hd < 1 || vd < 1) return fail("qkv_write: bad sizes");
  const int W = (nq + nkv) * hd + nkv * vd;
  const int threads = W >= 1024 ? 256 : 128;
  FLINT_DISPATCH_DTYPE(q_dtype, TQ, FLINT_DISPATCH_DTYPE(cache_dtype, TC,
      (launch_pdl(qkv_write_kernel<TQ, TC>, dim3(T), dim3(threads), 0, stream, qkv, n_partials, partial_stride, bias, pos,
                  slot, cos_t, sin_t, rot, interleaved, (TQ*)q_out, (TC*)k_cache, (TC*)v_cache, block_table, max_pages,
                  page_size, nq, nkv, hd, vd, v_keep, v_from, blend, status))));
  return check_launch("qkv_write");
}

extern "C" int flint_pool_write(const void* k_cache, const void* v_cache, void* pool_k, void* pool_v, int cache_dtype,
                                const int* block_table, int max_pages, int page_size, const int* pos, const int* slot,
                                int T, int nkv, int hd, int vd, int pool, int pool_slots, int* status, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (pool < 1 || pool_slots < 1 || (long long)pool_slots * pool < page_size)
    return fail("pool_write: %d means a page do not hold blocks of %d positions on pages of %d", pool_slots, pool, page_size);
  FLINT_DISPATCH_DTYPE(cache_dtype, TC,
      (launch_pdl(pool_write_kernel<TC>, dim3((unsigned)T, (unsigned)nkv), dim3(128), 0, stream, (const TC*)k_cache,
                  (const TC*)v_cache, (TC*)pool_k, (TC*)pool_v, block_table, max_pages, page_size, pos, slot, nkv, hd, vd,
                  pool, pool_slots, status)));
  return check_launch("pool_write");
}

// `scratch` must hold T * nq * n_splits * (vd + 2) floats when n_splits > 1; split_keys * n_splits must cover the
// most keys any row sees.  With a row list, T counts the listed rows and row_list[i] is the batch row of the i-th.
extern "C" int flint_sink_attention(const void* q, int q_dtype, const void* k_cache, const void* v_cache, int cache_dtype,
                                    const int* block_table, int max_pages, int page_size, const int* pos,
                                    const int* slot, void* out, int T, int nq, int nkv, int hd, int vd, int window,
                                    int keep_first, int run, const float* sinks, float scale, int split_keys,
                                    int n_splits, float* scratch, const int* row_list, const void* pool_k,
                                    const void* pool_v, int pool, int pool_slots, int sigmoid, float cap, const float* r1,
                                    const float* r2, const float* w_bias, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (hd < 1 || vd < 1 || hd > 256 || vd > 32 * MAX_DPL)
    return fail("sink_attention: head sizes %d (keys) and %d (values) are not supported (1 to 256)", hd, vd);
  if (nkv <= 0 || nq % nkv) return fail("sink_attention: %d query heads do not divide into %d kv heads", nq, nkv);
  if (n_splits < 1 || split_keys < 1) return fail("sink_attention: bad split (%d keys, %d splits)", split_keys, n_splits);
  if (n_splits > 1 && !scratch) return fail("sink_attention: splits need scratch memory");
  if (window < 0 || keep_first < 0 || run < 0 || (run > 0 && (window > 0 || keep_first > 0)))
    return fail("sink_attention: bad window (a run length excludes a window and kept first tokens)");
  if (pool < 0 || (pool > 0 && (window < 1 || keep_first > 0 || run > 0 || !pool_k || !pool_v || pool_slots < 1)))
    return fail("sink_attention: block means need a window, their storage, and no kept first tokens or runs");
  if (sigmoid && (sinks || (r1 == nullptr) != (r2 == nullptr)))
    return fail("sink_attention: weights without a softmax take no sink, and both numbers of the distance penalty or none");
  const SigmoidWeights sw = {sigmoid ? 1 : 0, cap, r1, r2, w_bias};
  const int elem = cache_dtype == FLINT_F32 ? 4 : 2;
  if ((hd % 8) == 0 && (((uintptr_t)k_cache) & 15)) return fail("sink_attention: the key cache must start on 16 bytes");
  (void)elem;
  const int G = nq / nkv;
  const int g_chunks = (G + GC - 1) / GC;
  const long long items = (long long)T * nkv * g_chunks * n_splits;
  const long long blocks = (items + WARPS - 1) / WARPS;
  if (blocks > 0x7fffffffLL) return fail("sink_attention: too many work items");
  const size_t smem = (size_t)WARPS * GC * hd * sizeof(float);
#define LAUNCH_D(TQ, TC, DPL)                                                                                         \
  launch_pdl(sink_attention_kernel<TQ, TC, TQ, DPL>, dim3((unsigned)blocks), dim3(WARPS * 32), smem, stream, (const TQ*)q, \
             (const TC*)k_cache, (const TC*)v_cache, block_table, max_pages, page_size, pos, slot, (TQ*)out, scratch, T, \
             nq, nkv, hd, vd, window, keep_first, run, sinks, scale, split_keys, n_splits, g_chunks, row_list,           \
             (const TC*)pool_k, (const TC*)pool_v, pool, pool_slots, sw)
#define LAUNCH(TQ, TC)                                                     \
  do {                                                                     \
    if (vd <= 64) LAUNCH_D(TQ, TC, 2);                                     \
    else if (vd <= 128) LAUNCH_D(TQ, TC, 4);                               \
    else LAUNCH_D(TQ, TC, 8);                                              \
  } while (0)
  FLINT_DISPATCH_DTYPE(q_dtype, TQ, FLINT_DISPATCH_DTYPE(cache_dtype, TC, LAUNCH(TQ, TC)));
#undef LAUNCH_D
#undef LAUNCH
  int rc = check_launch("sink_attention");
  if (rc || n_splits == 1) return rc;
  const int threads = vd >= 128 ? 128 : 64;
  FLINT_DISPATCH_DTYPE(q_dtype, TO,
      (launch_pdl(sink_combine_kernel<TO>, dim3((unsigned)((long long)T * nq)), dim3(threads), 0, stream,
                  (const float*)scratch, (TO*)out, vd, n_splits, nq, sinks, row_list, sigmoid ? 1 : 0)));
  return check_launch("sink_combine");
}

// tiles [n_tiles, 4] int32: first row, rows (up to 64), request slot, position of the first row; bfloat16 q, cache and
// out; head sizes in multiples of 16 up to 128.
extern "C" int flint_sink_attention_tiles(const void* q, const void* k_cache, const void* v_cache, const int* block_table,
                                          int max_pages, int page_size, const int* tiles, int n_tiles, void* out, int nq,
                                          int nkv, int hd, int vd, int window, int keep_first, int run,
                                          const float* sinks, float scale, const void* pool_k, const void* pool_v,
                                          int pool, int pool_slots, int sigmoid, float cap, const float* r1,
                                          const float* r2, const float* w_bias, cudaStream_t stream) {
  if (n_tiles <= 0) return 0;
  if (hd < 16 || vd < 16 || hd % 16 || vd % 16 || hd > 128 || vd > 128)
    return fail("sink_attention_tiles: head sizes %d and %d (multiples of 16 up to 128)", hd, vd);
  if (nkv <= 0 || nq % nkv) return fail("sink_attention_tiles: %d query heads do not divide into %d kv heads", nq, nkv);
  if (window < 0 || keep_first < 0 || page_size <= 0 || run < 0 || (run > 0 && (window > 0 || keep_first > 0)))
    return fail("sink_attention_tiles: bad window or page size");
  if (pool < 0 || (pool > 0 && (window < 1 || keep_first > 0 || run > 0 || !pool_k || !pool_v || pool_slots < 1)))
    return fail("sink_attention_tiles: block means need a window, their storage, and no kept first tokens or runs");
  if (sigmoid && (sinks || (r1 == nullptr) != (r2 == nullptr)))
    return fail("sink_attention_tiles: weights without a softmax take no sink, and both numbers of the penalty or none");
  const SigmoidWeights sw = {sigmoid ? 1 : 0, cap, r1, r2, w_bias};
  const __nv_bfloat16 *pk = (const __nv_bfloat16*)pool_k, *pv = (const __nv_bfloat16*)pool_v;
  if ((long long)n_tiles * nq > 0x7fffffffLL) return fail("sink_attention_tiles: too many work items");
  const size_t smem = 2 * ((size_t)MK * ((hd + 8) + (vd + 8)) * 2 + MK * sizeof(int));       // two stages
  const dim3 grid((unsigned)(n_tiles * nq)), block(128);
  static bool sized = false;
  if (!sized) {             // the larger form's two stages exceed the default limit of dynamic shared memory
    cudaFuncSetAttribute(sink_attention_mma_kernel<4, 8>, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024);
    cudaFuncSetAttribute(sink_attention_mma_kernel<8, 16>, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024);
    sized = true;
  }
  const __nv_bfloat16 *qq = (const __nv_bfloat16*)q, *kk = (const __nv_bfloat16*)k_cache, *vv = (const __nv_bfloat16*)v_cache;
  if (hd <= 64 && vd <= 64)
    launch_pdl(sink_attention_mma_kernel<4, 8>, grid, block, smem, stream, qq, kk, vv, block_table, max_pages, page_size, tiles,
               (__nv_bfloat16*)out, nq, nkv, hd, vd, window, keep_first, run, sinks, scale, pk, pv, pool, pool_slots, sw);
  else
    launch_pdl(sink_attention_mma_kernel<8, 16>, grid, block, smem, stream, qq, kk, vv, block_table, max_pages, page_size, tiles,
               (__nv_bfloat16*)out, nq, nkv, hd, vd, window, keep_first, run, sinks, scale, pk, pv, pool, pool_slots, sw);
  return check_launch("sink_attention_tiles");
}

extern "C" const char* flint_attention_sink_last_error() { return g_error; }
