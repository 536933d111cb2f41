// Routing for a mixture of experts: router logits with sparsemixer top-2 selection or a softmax choice of the
// top k limited to groups, and the plan that sorts token rows by expert for the grouped products.
//
// The reference has no mixture of experts (its feed-forward is dense:
// crates/thuban_model/src/ops/mlp.rs:24-79); these kernels have no counterpart there.
// Router logits, the mask threshold and both softmaxes are float32 in every mode.
#include <math.h>
#include <stdarg.h>
#include "common.cuh"
#include "router_select.cuh"

using namespace flint;

namespace {
constexpr int MAX_E = 256;

// One block per TT tokens.  The tokens' rows are staged in shared memory; each warp takes
// experts warp, warp+16, ... and computes their logits for all TT tokens while reading the
// router row once with 16-byte loads; then one thread per token does the selection:
//   i1 = argmax s (lowest index on ties), m1 = s[i1]
//   keep_j = !((m1 - s_j) / max(|s_j|, m1) > 2 eps);  g1 = e^{s_i1 - m1} / sum_{keep} e^{s_j - m1}
//   the same again over s without i1 for (i2, g2); the gates are not renormalised.
constexpr int TT = 4;
constexpr int ROUTER_WARPS = 16;

template <typename TW> struct Vec;                       // 16 bytes of a weight row
template <> struct Vec<float> { static constexpr int N = 4; };
template <> struct Vec<__nv_bfloat16> { static constexpr int N = 8; };

__device__ __forceinline__ void load_vec(const float* p, float* f) {
  const float4 a = *reinterpret_cast<const float4*>(p);
  f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w;
}
__device__ __forceinline__ void load_vec(const __nv_bfloat16* p, float* f) {
  const uint4 a = *reinterpret_cast<const uint4*>(p);
  const uint32_t w[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    f[2 * i] = __uint_as_float(w[i] << 16);
    f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
  }
}

// The float32 router logits of the block's TT tokens into s_all [TT, E] (shared memory; xs holds the staged rows).
template <typename TW>
__device__ __forceinline__ void block_router_logits(const float* __restrict__ x, const TW* __restrict__ wr, float* xs,
                                                    float* s_all, int t0, int nt, int H, int E, int vec_ok) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (vec_ok) {        // rows are staged with 16-byte loads, several in flight per thread
    const int n4 = TT * H / 4, live4 = nt * H / 4;
    const float4* src = reinterpret_cast<const float4*>(x + (size_t)t0 * H);
    float4* dst = reinterpret_cast<float4*>(xs);
#pragma unroll 8
    for (int i = threadIdx.x; i < n4; i += blockDim.x)
      dst[i] = i < live4 ? src[i] : make_float4(0.f, 0.f, 0.f, 0.f);
  } else {
    for (int i = threadIdx.x; i < TT * H; i += blockDim.x) xs[i] = i < nt * H ? x[(size_t)t0 * H + i] : 0.f;
  }
  __syncthreads();
  constexpr int VN = Vec<TW>::N;
  constexpr int EW = 4;            // experts a warp works side by side: their weight loads are in flight together
  for (int e0 = warp * EW; e0 < E; e0 += ROUTER_WARPS * EW) {
    float a[EW][TT];
#pragma unroll
    for (int k = 0; k < EW; ++k)
#pragma unroll
      for (int tt = 0; tt < TT; ++tt) a[k][tt] = 0.f;
    if (vec_ok) {
#pragma unroll 2
      for (int d = lane * VN; d < H; d += 32 * VN) {
        float wv[EW][VN];
#pragma unroll
        for (int k = 0; k < EW; ++k) {
          if (e0 + k < E) load_vec(wr + (size_t)(e0 + k) * H + d, wv[k]);
          else
#pragma unroll
            for (int i = 0; i < VN; ++i) wv[k][i] = 0.f;
        }
#pragma unroll
        for (int tt = 0; tt < TT; ++tt) {
          float xv[VN];                       // 16-byte reads of the staged row: no bank conflicts
#pragma unroll
          for (int i = 0; i < VN; i += 4) load_vec(xs + tt * H + d + i, xv + i);
#pragma unroll
          for (int k = 0; k < EW; ++k)
#pragma unroll
            for (int i = 0; i < VN; ++i) a[k][tt] = fmaf(xv[i], wv[k][i], a[k][tt]);
        }
      }
    } else {
      for (int d = lane; d < H; d += 32) {
#pragma unroll
        for (int k = 0; k < EW; ++k) {
          const float wv = e0 + k < E ? to_f32(wr[(size_t)(e0 + k) * H + d]) : 0.f;
#pragma unroll
          for (int tt = 0; tt < TT; ++tt) a[k][tt] = fmaf(xs[tt * H + d], wv, a[k][tt]);
        }
      }
    }
#pragma unroll
    for (int k = 0; k < EW; ++k)
#pragma unroll
      for (int tt = 0; tt < TT; ++tt) {
        const float v = warp_sum(a[k][tt]);
        if (lane == 0 && e0 + k < E) s_all[tt * E + e0 + k] = v;
      }
  }
  __syncthreads();
}

template <typename TW>
__global__ void __launch_bounds__(ROUTER_WARPS * 32)
router_sparsemixer_kernel(const float* __restrict__ x, const TW* __restrict__ wr, float eps,
                          int* __restrict__ expert_ids, float* __restrict__ gates,
                          float* __restrict__ logits_out, int T, int H, int E, int vec_ok) {
  extern __shared__ float smem[];   // TT rows of x, then TT x E logits
  float* xs = smem;
  float* s_all = smem + (size_t)TT * H;
  const int t0 = blockIdx.x * TT;
  const int nt = min(TT, T - t0);
  block_router_logits<TW>(x, wr, xs, s_all, t0, nt, H, E, vec_ok);
  if (threadIdx.x >= nt) return;
  const int t = t0 + threadIdx.x;
  const float* s = s_all + threadIdx.x * E;
  if (logits_out)
    for (int e = 0; e < E; ++e) logits_out[(size_t)t * E + e] = s[e];
  int sel[2];
  float gate[2];
  int excluded = -1;
  for (int r = 0; r < 2; ++r) {
    float m = -INFINITY;
    int im = 0;
    for (int e = 0; e < E; ++e)
      if (e != excluded && s[e] > m) { m = s[e]; im = e; }
    float denom = 0.f;
    for (int e = 0; e < E; ++e) {
      if (e == excluded) continue;
      const float factor = fmaxf(fabsf(s[e]), m);
      const bool masked = ((m - s[e]) / factor) > 2.0f * eps;
      if (!masked) denom += expf(s[e] - m);
    }
    sel[r] = im;
    gate[r] = 1.0f / denom;   // e^{m - m} / denom
    excluded = im;
  }
  expert_ids[2 * t] = sel[0];
  expert_ids[2 * t + 1] = sel[1];
  gates[2 * t] = gate[0];
  gates[2 * t + 1] = gate[1];
}

// Softmax router with a choice limited to groups: s = softmax(logits); the experts form n_groups equal groups of
// neighbours, a group scores as its best member, only members of the `keep` best groups may be chosen, and the
// `top` best of those are (lowest index first among equals).  Gates: s_e / (sum of the chosen s + 1e-20) * scale.
// One warp per token does the selection (a lane holds every 32nd expert); everything is float32.
constexpr int MAX_TOP = ROUTER_MAX_TOP;
template <typename TW>
__global__ void __launch_bounds__(ROUTER_WARPS * 32)
router_topk_kernel(const float* __restrict__ x, const TW* __restrict__ wr, int top, int n_groups, int keep,
                   float out_scale, int* __restrict__ expert_ids, float* __restrict__ gates,
                   float* __restrict__ logits_out, int T, int H, int E, int vec_ok) {
  extern __shared__ float smem[];   // TT rows of x, then TT x E logits (turned into scores in place)
  float* xs = smem;
  float* s_all = smem + (size_t)TT * H;
  pdl_launch();
  pdl_wait();
  const int t0 = blockIdx.x * TT;
  const int nt = min(TT, T - t0);
  block_router_logits<TW>(x, wr, xs, s_all, t0, nt, H, E, vec_ok);
  // one warp per token
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (warp >= nt) return;
  const int t = t0 + warp;
  float* s = s_all + warp * E;
  if (logits_out)
    for (int e = lane; e < E; e += 32) logits_out[(size_t)t * E + e] = s[e];
  select_topk_by_warp(s, lane, E, top, n_groups, keep, out_scale, expert_ids + (size_t)t * top, gates + (size_t)t * top);
}

// One block.  expert_ids [T*top] -> per-expert counts, offsets (exclusive scan), the sorted row
// of every (token, choice) and the tile map for the grouped products.
__global__ void moe_plan_kernel(const int* __restrict__ expert_ids, int n_assign, int E,
                                int tile_rows, int* __restrict__ counts, int* __restrict__ offsets,
                                int* __restrict__ row_of, int* __restrict__ token_of,
                                int* __restrict__ tile_expert, int* __restrict__ tile_row0,
                                int* __restrict__ n_tiles, int max_tiles, int top) {
  __shared__ int cnt[MAX_E];
  __shared__ int off[MAX_E + 1];
  pdl_launch();
  pdl_wait();
  for (int e = threadIdx.x; e < E; e += blockDim.x) cnt[e] = 0;
  __syncthreads();
  // rank of each assignment inside its expert (the order inside an expert has no effect on
  // any result: rows are independent in the products and are added back per token)
  for (int a = threadIdx.x; a < n_assign; a += blockDim.x) row_of[a] = atomicAdd(&cnt[expert_ids[a]], 1);
  __syncthreads();
  if (threadIdx.x == 0) {
    int run = 0, tiles = 0;
    for (int e = 0; e < E; ++e) {
      off[e] = run;
      counts[e] = cnt[e];
      offsets[e] = run;
      for (int r = 0; r < cnt[e]; r += tile_rows) {
        if (tiles < max_tiles) {
          tile_expert[tiles] = e;
          tile_row0[tiles] = run + r;
        }
        ++tiles;
      }
      run += cnt[e];
    }
    off[E] = run;
    offsets[E] = run;
    *n_tiles = tiles < max_tiles ? tiles : max_tiles;
  }
  __syncthreads();
  for (int a = threadIdx.x; a < n_assign; a += blockDim.x) {
    const int row = off[expert_ids[a]] + row_of[a];
    row_of[a] = row;
    token_of[row] = a / top;
  }
}

// Few assignments (decode): the plan and the gather of the rows in one launch.  Every block works the
// (tiny) plan out again in shared memory, with ranks by position so that all blocks agree; block r then
// copies the row of its token to sorted row r, and block 0 also writes the plan out.
constexpr int DISPATCH_MAX = 256;      // assignments
__global__ void __launch_bounds__(256)
moe_dispatch_kernel(const int* __restrict__ expert_ids, int n_assign, int E, int tile_rows,
                    int* __restrict__ counts, int* __restrict__ offsets, int* __restrict__ row_of,
                    int* __restrict__ token_of, int* __restrict__ tile_expert, int* __restrict__ tile_row0,
                    int* __restrict__ n_tiles, int max_tiles, const uint4* __restrict__ x,
                    uint4* __restrict__ xs, int row_vecs, int top) {
  __shared__ int ids[DISPATCH_MAX];
  __shared__ int cnt[MAX_E];
  __shared__ int off[MAX_E + 1];
  __shared__ int my_token;
  pdl_launch();
  pdl_wait();
  const int tid = threadIdx.x;
  if (tid < n_assign) ids[tid] = expert_ids[tid];
  __syncthreads();
  if (tid < E) {
    int c = 0;
    for (int a = 0; a < n_assign; ++a) c += ids[a] == tid;
    cnt[tid] = c;
  }
  int rank = 0;                       // assignments before this one that chose the same expert
  if (tid < n_assign)
    for (int a = 0; a < tid; ++a) rank += ids[a] == ids[tid];
  __syncthreads();
  if (tid == 0) {
    const bool out = blockIdx.x == 0;
    int run = 0, tiles = 0;
    for (int e = 0; e < E; ++e) {
      off[e] = run;
      if (out) {
        counts[e] = cnt[e];
        offsets[e] = run;
        for (int r = 0; r < cnt[e]; r += tile_rows) {
          if (tiles < max_tiles) {
            tile_expert[tiles] = e;
            tile_row0[tiles] = run + r;
          }
          ++tiles;
        }
      }
      run += cnt[e];
    }
    off[E] = run;
    if (out) {
      offsets[E] = run;
      *n_tiles = tiles < max_tiles ? tiles : max_tiles;
    }
  }
  __syncthreads();
  if (tid < n_assign) {
    const int row = off[ids[tid]] + rank;
    if (blockIdx.x == 0) {
      row_of[tid] = row;
      token_of[row] = tid / top;
    }
    if (row == (int)blockIdx.x) my_token = tid / top;
  }
  __syncthreads();
  const uint4* src = x + (size_t)my_token * row_vecs;
  uint4* dst = xs + (size_t)blockIdx.x * row_vecs;
  for (int i = tid; i < row_vecs; i += blockDim.x) dst[i] = src[i];
}
}  // namespace

extern "C" int flint_router_sparsemixer(const float* x, const void* wr, int w_dtype, float eps,
                                        int* expert_ids, float* gates, float* logits_out, int T,
                                        int H, int E, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (E < 2 || E > MAX_E) return fail("router: %d experts (supported: 2..%d)", E, MAX_E);
  const size_t smem = ((size_t)TT * H + (size_t)TT * E) * sizeof(float);
  if (smem > 200 * 1024) return fail("router: width %d is too large for the staging buffer", H);
  const int blocks = (T + TT - 1) / TT;
  // 16-byte loads of the router rows need rows that start on 16 bytes
  const int vec_ok = (H % 8 == 0) && (((uintptr_t)wr & 15) == 0);
  static bool configured[2] = {false, false};
  if (smem > 48 * 1024 && !configured[w_dtype ? 1 : 0]) {
    cudaError_t e = w_dtype == FLINT_F32
        ? cudaFuncSetAttribute(router_sparsemixer_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024)
        : cudaFuncSetAttribute(router_sparsemixer_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    if (e != cudaSuccess) return fail("router: cannot raise shared memory: %s", cudaGetErrorString(e));
    configured[w_dtype ? 1 : 0] = true;
  }
  FLINT_DISPATCH_DTYPE(w_dtype, TW,
      (router_sparsemixer_kernel<TW><<<blocks, ROUTER_WARPS * 32, smem, stream>>>(
          x, (const TW*)wr, eps, expert_ids, gates, logits_out, T, H, E, vec_ok)));
  return check_launch("router_sparsemixer");
}

// x [T, H] float32, wr [E, H]; expert_ids and gates [T, top].
extern "C" int flint_router_topk(const float* x, const void* wr, int w_dtype, int top, int n_groups, int keep,
                                 float out_scale, int* expert_ids, float* gates, float* logits_out, int T, int H, int E,
                                 cudaStream_t stream) {
  if (T <= 0) return 0;
  if (E < 1 || E > MAX_E) return fail("router: %d experts (supported: 1..%d)", E, MAX_E);
  if (top < 1 || top > MAX_TOP || top > E) return fail("router: %d choices of %d experts (supported: 1..%d)", top, E, MAX_TOP);
  if (n_groups < 1 || n_groups > 64 || E % n_groups) return fail("router: %d experts do not form %d equal groups (up to 64)", E, n_groups);
  if (keep < 1 || keep > n_groups) return fail("router: %d of %d groups kept", keep, n_groups);
  if (keep * (E / n_groups) < top) return fail("router: %d kept groups of %d experts cannot give %d choices", keep, E / n_groups, top);
  const size_t smem = ((size_t)TT * H + (size_t)TT * E) * sizeof(float);
  if (smem > 200 * 1024) return fail("router: width %d is too large for the staging buffer", H);
  const int blocks = (T + TT - 1) / TT;
  const int vec_ok = (H % 8 == 0) && (((uintptr_t)wr & 15) == 0) && (((uintptr_t)x & 15) == 0);
  static bool configured[2] = {false, false};
  if (smem > 48 * 1024 && !configured[w_dtype ? 1 : 0]) {
    cudaError_t e = w_dtype == FLINT_F32
        ? cudaFuncSetAttribute(router_topk_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024)
        : cudaFuncSetAttribute(router_topk_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    if (e != cudaSuccess) return fail("router: cannot raise shared memory: %s", cudaGetErrorString(e));
    configured[w_dtype ? 1 : 0] = true;
  }
  FLINT_DISPATCH_DTYPE(w_dtype, TW,
      (launch_pdl(router_topk_kernel<TW>, dim3(blocks), dim3(ROUTER_WARPS * 32), smem, stream, x, (const TW*)wr, top,
                  n_groups, keep, out_scale, expert_ids, gates, logits_out, T, H, E, vec_ok)));
  return check_launch("router_topk");
}

// Upper bound of row tiles for n_assign rows over E experts.
// --------------------------------------------------------------------------- sigmoid router
// Scores s_e = sigmoid(<x, Wr[e]>) in float32 over the first E rows of Wr; the `top` largest are chosen (the lower
// index among equals) with their scores as they are.  Rows E .. E + X - 1 of Wr are not experts but gates of
// always-on parts: their sigmoids go to weights[:, top:], and weights[:, :top] is 1 (the chosen experts' scores
// scale their inputs, so their outputs are added as they are).  A warp takes RT tokens and reads every weight
// row once for all of them.
constexpr int RT = 4;
template <typename TW>
__global__ void __launch_bounds__(128)
router_sigmoid_kernel(const float* __restrict__ x, const TW* __restrict__ wr, int T, int H, int E, int X, int top,
                      int* __restrict__ expert_ids, float* __restrict__ scores, float* __restrict__ weights,
                      float* __restrict__ logits_out) {
  extern __shared__ float smem[];            // per warp: RT * (E + X) logits
  pdl_launch();
  pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t0 = (blockIdx.x * 4 + warp) * RT;
  if (t0 >= T) return;
  const int nt = min(RT, T - t0), R = E + X;
  float* z = smem + warp * RT * R;
  for (int e = 0; e < R; ++e) {
    float acc[RT];
#pragma unroll
    for (int r = 0; r < RT; ++r) acc[r] = 0.f;
    const TW* w = wr + (size_t)e * H;
    for (int d = lane; d < H; d += 32) {
      const float wv = to_f32(w[d]);
#pragma unroll
      for (int r = 0; r < RT; ++r)
        if (r < nt) acc[r] = fmaf(x[(size_t)(t0 + r) * H + d], wv, acc[r]);
    }
#pragma unroll
    for (int r = 0; r < RT; ++r) {
      const float v = warp_sum(acc[r]);
      if (lane == 0 && r < nt) z[r * R + e] = v;
    }
  }
  __syncwarp();
  for (int r = 0; r < nt; ++r) {
    const int t = t0 + r;
    float* zr = z + r * R;
    if (logits_out)
      for (int e = lane; e < R; e += 32) logits_out[(size_t)t * R + e] = zr[e];
    __syncwarp();
    select_sigmoid_by_warp(zr, lane, E, X, top, expert_ids + (size_t)t * top, scores + (size_t)t * top,
                           weights + (size_t)t * (top + X));
  }
}

extern "C" int flint_router_sigmoid(const float* x, const void* wr, int w_dtype, int E, int X, int top, int* expert_ids,
                                    float* scores, float* weights, float* logits_out, int T, int H,
                                    cudaStream_t stream) {
  if (T <= 0) return 0;
  if (E < 1 || X < 0 || top < 1 || top > E) return fail("router_sigmoid: %d of %d experts (+%d gates) is not supported", top, E, X);
  const size_t smem = (size_t)4 * RT * (E + X) * sizeof(float);
  if (smem > 48 * 1024) return fail("router_sigmoid: too many experts (%d)", E);
  const unsigned blocks = (unsigned)((T + 4 * RT - 1) / (4 * RT));
  FLINT_DISPATCH_DTYPE(w_dtype, TW,
      launch_pdl(router_sigmoid_kernel<TW>, dim3(blocks), dim3(128), smem, stream, x, (const TW*)wr, T, H, E, X, top,
                 expert_ids, scores, weights, logits_out));
  return check_launch("router_sigmoid");
}

// The grouped sigmoid router (select_sigmoid_grouped_by_warp) as a kernel of its own: a warp takes RT tokens, walks
// the experts' weight rows once for all of them, then selects token by token.
template <typename TW>
__global__ void __launch_bounds__(128)
router_sigmoid_grouped_kernel(const float* __restrict__ x, const TW* __restrict__ wr, const float* __restrict__ correction,
                              int T, int H, int E, int top, int n_groups, int keep, int normalize, float out_scale,
                              int* __restrict__ expert_ids, float* __restrict__ gates, float* __restrict__ logits_out) {
  extern __shared__ float smem[];            // per warp: RT * E logits, then E choice scores
  pdl_launch();
  pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t0 = (blockIdx.x * 4 + warp) * RT;
  if (t0 >= T) return;
  const int nt = min(RT, T - t0);
  float* z = smem + warp * (RT + 1) * E;
  float* c = z + RT * E;
  for (int e = 0; e < E; ++e) {
    float acc[RT];
#pragma unroll
    for (int r = 0; r < RT; ++r) acc[r] = 0.f;
    const TW* w = wr + (size_t)e * H;
    for (int d = lane; d < H; d += 32) {
      const float wv = to_f32(w[d]);
#pragma unroll
      for (int r = 0; r < RT; ++r)
        if (r < nt) acc[r] = fmaf(x[(size_t)(t0 + r) * H + d], wv, acc[r]);
    }
#pragma unroll
    for (int r = 0; r < RT; ++r) {
      const float v = warp_sum(acc[r]);
      if (lane == 0 && r < nt) z[r * E + e] = v;
    }
  }
  __syncwarp();
  for (int r = 0; r < nt; ++r) {
    const int t = t0 + r;
    float* zr = z + r * E;
    if (logits_out)
      for (int e = lane; e < E; e += 32) logits_out[(size_t)t * E + e] = zr[e];
    __syncwarp();
    select_sigmoid_grouped_by_warp(zr, c, correction, lane, E, top, n_groups, keep, normalize, out_scale,
                                   expert_ids + (size_t)t * top, gates + (size_t)t * top);
    __syncwarp();
  }
}

extern "C" int flint_router_sigmoid_grouped(const float* x, const void* wr, int w_dtype, const float* correction, int E,
                                            int top, int n_groups, int keep, int normalize, float out_scale,
                                            int* expert_ids, float* gates, float* logits_out, int T, int H,
                                            cudaStream_t stream) {
  if (T <= 0) return 0;
  if (E < 1 || top < 1 || top > E || top > 32) return fail("router_sigmoid_grouped: %d of %d experts is not supported", top, E);
  if (n_groups < 1 || n_groups > 64 || E % n_groups || keep < 1 || keep > n_groups || keep * (E / n_groups) < top)
    return fail("router_sigmoid_grouped: %d of %d groups of %d experts cannot give %d a token", keep, n_groups, E, top);
  const size_t smem = (size_t)4 * (RT + 1) * E * sizeof(float);
  if (smem > 48 * 1024) return fail("router_sigmoid_grouped: too many experts (%d)", E);
  const unsigned blocks = (unsigned)((T + 4 * RT - 1) / (4 * RT));
  FLINT_DISPATCH_DTYPE(w_dtype, TW,
      launch_pdl(router_sigmoid_grouped_kernel<TW>, dim3(blocks), dim3(128), smem, stream, x, (const TW*)wr, correction, T, H,
                 E, top, n_groups, keep, normalize, out_scale, expert_ids, gates, logits_out));
  return check_launch("router_sigmoid_grouped");
}

extern "C" int flint_moe_max_tiles(int n_assign, int E, int tile_rows) {
  return n_assign / tile_rows + (E < n_assign ? E : n_assign);
}

extern "C" int flint_moe_plan(const int* expert_ids, int n_assign, int E, int tile_rows, int* counts,
                              int* offsets, int* row_of, int* token_of, int* tile_expert,
                              int* tile_row0, int* n_tiles, int max_tiles, int top, cudaStream_t stream) {
  if (n_assign <= 0) return 0;
  if (top < 1) return fail("moe_plan: %d choices a token", top);
  if (E < 1 || E > MAX_E) return fail("moe_plan: %d experts (supported: 1..%d)", E, MAX_E);
  if (tile_rows <= 0) return fail("moe_plan: bad tile size %d", tile_rows);
  if (max_tiles < flint_moe_max_tiles(n_assign, E, tile_rows))
    return fail("moe_plan: tile map of %d entries is too small", max_tiles);
  launch_pdl(moe_plan_kernel, dim3(1), dim3(1024), 0, stream, expert_ids, n_assign, E, tile_rows, counts, offsets, row_of,
                                          token_of, tile_expert, tile_row0, n_tiles, max_tiles, top);
  return check_launch("moe_plan");
}

// The plan of flint_moe_plan and xs[r, :] = x[token_of[r], :] in one launch, for up to 256 assignments and rows
// of a multiple of 16 bytes (x and xs 16-byte aligned).
extern "C" int flint_moe_dispatch(const int* expert_ids, int n_assign, int E, int tile_rows, int* counts,
                                  int* offsets, int* row_of, int* token_of, int* tile_expert, int* tile_row0,
                                  int* n_tiles, int max_tiles, const void* x, void* xs, int row_bytes, int top,
                                  cudaStream_t stream) {
  if (n_assign <= 0) return 0;
  if (top < 1) return fail("moe_dispatch: %d choices a token", top);
  if (n_assign > DISPATCH_MAX) return fail("moe_dispatch: %d assignments (up to %d)", n_assign, DISPATCH_MAX);
  if (E < 1 || E > MAX_E) return fail("moe_dispatch: %d experts (supported: 1..%d)", E, MAX_E);
  if (tile_rows <= 0) return fail("moe_dispatch: bad tile size %d", tile_rows);
  if (max_tiles < flint_moe_max_tiles(n_assign, E, tile_rows))
    return fail("moe_dispatch: tile map of %d entries is too small", max_tiles);
  if (row_bytes <= 0 || (row_bytes & 15) || ((uintptr_t)x & 15) || ((uintptr_t)xs & 15))
    return fail("moe_dispatch: rows must be a multiple of 16 bytes and 16-byte aligned");
  launch_pdl(moe_dispatch_kernel, dim3(n_assign), dim3(256), 0, stream, expert_ids, n_assign, E, tile_rows, counts,
             offsets, row_of, token_of, tile_expert, tile_row0, n_tiles, max_tiles, (const uint4*)x, (uint4*)xs,
             row_bytes / 16, top);
  return check_launch("moe_dispatch");
}

extern "C" const char* flint_moe_last_error() { return g_error; }
