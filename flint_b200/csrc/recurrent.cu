// Kernels of mixers that carry state from token to token: a short causal convolution over time, the recurrence of
// the gated delta rule and of a state-space model with a scalar decay per head, and what surrounds them.
//
// Short convolution.  y[t, c] = act(b[c] + sum_j w[c, j] u[t - taps + 1 + j, c]) over the rows of one request, zeros
// before its first position.  The inputs of earlier steps come from the request's state, taps - 1 rows: the input at
// position p lives in state row p mod (taps - 1).  The convolution's kernel only reads the state; a second kernel,
// launched behind it, stores the inputs of every request's last taps - 1 rows of the step.  So every row of the batch
// is worked independently, and no row of the state is read and written in one launch.
//
// Recurrence.  Per request and head a float32 matrix S [D, V] (key dims by value dims) lives in the state slab.
//   gated delta rule:  S <- diag(g_t) S;  u = beta_t (v_t - S^T k_t);  S <- S + k_t u^T;  o_t = S^T q_t
//   state space:       S <- a_t S + k_t (dt_t v_t)^T;                                     o_t = S^T q_t + skip v_t
// (for the state-space form k is the input matrix B and q the read-out C).  Columns of S are independent, so a block
// takes a request, a head and a run of columns; a column is held by 1, 2, 4 or 8 neighbouring lanes, 32 rows each in
// registers, which meet by shuffles for the two dot products.  Tokens are walked one by one in float32 whatever the
// cut of the prompt, their operands staged through shared memory a few tokens at a time by asynchronous copies in
// two alternating stages, so a portion, a single token and a whole prompt give the same bits from the same state.
//
// The reference keeps recurrent state per sequence outside the paged pool and runs its delta rule token by token
// as well (crates/thuban_architectures/src/qwen35/state.rs:5-55).
#include <math.h>
#include <stdarg.h>
#include "common.cuh"

using namespace flint;

namespace {

__device__ __forceinline__ float sigmoidf_(float x) { return 1.0f / (1.0f + expf(-x)); }
__device__ __forceinline__ float siluf_(float x) { return x / (1.0f + expf(-x)); }
__device__ __forceinline__ float softplusf_(float x) { return x > 20.0f ? x : log1pf(expf(x)); }

// true if row t - d of the batch is the same request's token d positions earlier
__device__ __forceinline__ bool same_request(const int* pos, const int* slot, int t, int d, int T) {
  const int r = t - d;
  return r >= 0 && r < T && slot[r] == slot[t] && pos[r] == pos[t] - d;
}

// ------------------------------------------------------------------------------------------- short convolution
// u: float32 rows of `in_stride` floats, the convolved channels start at column col0.  Grid: (rows, blocks of channels).
__global__ void short_conv_kernel(const float* __restrict__ u, long long in_stride, int col0, const float* __restrict__ w,
                                  const float* __restrict__ bias, int act, const int* __restrict__ pos,
                                  const int* __restrict__ slot, const float* __restrict__ ring, long long ring_stride,
                                  float* __restrict__ y, int T, int C, int taps) {
  pdl_launch();
  pdl_wait();
  const int t = blockIdx.x;
  const int p = pos[t], R = taps - 1;
  // how many of the taps - 1 earlier inputs are rows of this batch
  int have = 0;
  while (have < taps - 1 && same_request(pos, slot, t, have + 1, T)) ++have;
  const float* mine = ring + (size_t)slot[t] * ring_stride;
  const float* row = u + (size_t)t * in_stride + col0;
  for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < C; c += gridDim.y * blockDim.x) {
    float acc = bias ? bias[c] : 0.f;
    for (int d = taps - 1; d >= 1; --d) {          // oldest first: the order of the sum does not depend on the cut
      const int q = p - d;
      float x = 0.f;
      if (q >= 0) x = d <= have ? row[c - (long long)d * in_stride] : mine[(size_t)(q % R) * C + c];
      acc = fmaf(w[(size_t)c * taps + (taps - 1 - d)], x, acc);
    }
    acc = fmaf(w[(size_t)c * taps + taps - 1], row[c], acc);
    y[(size_t)t * C + c] = act == 1 ? siluf_(acc) : acc;
  }
}

// The inputs that outlive the step: a row that is among the last taps - 1 of its request's rows stores its input.
__global__ void short_conv_keep_kernel(const float* __restrict__ u, long long in_stride, int col0,
                                       const int* __restrict__ pos, const int* __restrict__ slot, float* __restrict__ ring,
                                       long long ring_stride, int T, int C, int taps) {
  pdl_launch();
  pdl_wait();
  const int t = blockIdx.x;
  if (same_request(pos, slot, t, -(taps - 1), T)) return;
  float* mine = ring + (size_t)slot[t] * ring_stride + (size_t)(pos[t] % (taps - 1)) * C;
  const float* row = u + (size_t)t * in_stride + col0;
  for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < C; c += gridDim.y * blockDim.x) mine[c] = row[c];
}

// ------------------------------------------------------------------------------------------- gated delta rule: operands
// y [T, 2 G D + H V]: q | k | v after the convolution.  q and k become unit vectors per head (q times D^(-1/2));
// beta = sigmoid(b); decay[t, h, d] = exp(-exp(A_log[h]) softplus(a[t, h, d] + dt_bias[h, d])).  One block per row.
__global__ void delta_prepare_kernel(const float* __restrict__ y, long long y_stride, const float* __restrict__ b,
                                     long long b_stride, const float* __restrict__ a, const float* __restrict__ dt_bias,
                                     const float* __restrict__ a_log, float* __restrict__ qk, float* __restrict__ decay,
                                     float* __restrict__ beta, int H, int G, int D, float unit_eps) {
  pdl_launch();
  pdl_wait();
  const int t = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  const float* row = y + (size_t)t * y_stride;
  const float q_scale = rsqrtf((float)D);
  for (int g = warp; g < 2 * G; g += nw) {            // heads of q, then heads of k
    const float* src = row + (size_t)g * D;
    float ss = 0.f;
    for (int d = lane; d < D; d += 32) ss = fmaf(src[d], src[d], ss);
    ss = warp_sum(ss);
    const float inv = (1.0f / sqrtf(ss + unit_eps)) * (g < G ? q_scale : 1.0f);
    for (int d = lane; d < D; d += 32) qk[(size_t)t * 2 * G * D + (size_t)g * D + d] = src[d] * inv;
  }
  for (int e = threadIdx.x; e < H * D; e += blockDim.x) {
    const float rate = expf(a_log[e / D]);
    decay[(size_t)t * H * D + e] = expf(-rate * softplusf_(a[(size_t)t * H * D + e] + dt_bias[e]));
  }
  for (int h = threadIdx.x; h < H; h += blockDim.x) beta[(size_t)t * H + h] = sigmoidf_(b[(size_t)t * b_stride + h]);
}

// dt = softplus(raw + dt_bias); decay = exp(-exp(A_log) dt); raw [T, H] with a row stride.
__global__ void ssd_prepare_kernel(const float* __restrict__ raw, long long raw_stride, const float* __restrict__ dt_bias,
                                   const float* __restrict__ a_log, float* __restrict__ dt, float* __restrict__ decay,
                                   int T, int H) {
  pdl_launch();
  pdl_wait();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= T * H) return;
  const int t = i / H, h = i % H;
  const float d = softplusf_(raw[(size_t)t * raw_stride + h] + dt_bias[h]);
  dt[i] = d;
  decay[i] = expf(-expf(a_log[h]) * d);
}

// ------------------------------------------------------------------------------------------- the recurrence
constexpr int RPT = 32;          // rows of S a thread holds
constexpr int SCAN_THREADS = 128;

__device__ __forceinline__ void copy4(float* dst, const float* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}

__device__ __forceinline__ void copy16(float* dst, const float* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}

constexpr int SEG = RPT + 4;     // floats between the rows of neighbouring lanes of a column: their 16-byte reads miss each other's banks

// TPC: threads per column (D <= 32 TPC).  DELTA: the gated delta rule (a decay per key channel, the write corrected
// by what the state already returns for the key), else the state-space form (one decay per head, plain write).
// q, k [T, G D] and v [T, H V] are float32 views with row strides; decay [T, H D] (DELTA) or [T, H]; w1 [T, H]: beta
// (DELTA) or dt; skip [H] or null.  seq_start [n_seq + 1] or null (row e is request e).  Grid: (column blocks, H, n_seq).
// VEC: every row of q, k, v and decay starts on a 16-byte boundary and D and V are multiples of 4, so the operands are
// staged 16 bytes a copy; else 4 bytes a copy.  Both leave the same numbers in the same places.
template <int TPC, bool DELTA, bool VEC>
__global__ void __launch_bounds__(SCAN_THREADS)
recurrence_scan_kernel(const float* __restrict__ q, long long q_stride, const float* __restrict__ k, long long k_stride,
                       const float* __restrict__ v, long long v_stride, const float* __restrict__ decay,
                       const float* __restrict__ w1, const float* __restrict__ skip, const int* __restrict__ slot,
                       const int* __restrict__ seq_start, float* __restrict__ state, long long state_stride,
                       float* __restrict__ o, int H, int G, int D, int V, int TB) {
  extern __shared__ __align__(16) float sm[];
  constexpr int DP = TPC * SEG;                  // floats of a staged vector of key dims: lane s of a column reads from s SEG
  constexpr int NV = DELTA ? 3 : 2;              // staged vectors a token: q, k (and the decay per channel)
  constexpr int COLS = SCAN_THREADS / TPC;       // columns a block takes
  const int tid = threadIdx.x, sub = tid % TPC, col = blockIdx.x * COLS + tid / TPC;
  const int h = blockIdx.y, e = blockIdx.z, kh = h / (H / G);
  const int r0 = seq_start ? seq_start[e] : e, r1 = seq_start ? seq_start[e + 1] : e + 1;
  if (r1 <= r0) return;
  // a stage: TB tokens of q, k (and decay per channel), the columns' values, and two numbers a token
  const int per_tok = NV * DP + COLS + 4;        // a multiple of 4: the operands are read as float4
  float* stage[2] = {sm, sm + (size_t)TB * per_tok};
  for (int i = tid; i < 2 * TB * per_tok; i += SCAN_THREADS) {      // dims beyond D: q = k = 0, decay = 1
    const int w = i % per_tok;
    sm[i] = (DELTA && w >= 2 * DP && w < 3 * DP) ? 1.f : 0.f;
  }
  __syncthreads();
  pdl_wait();
  const bool live = col < V;
  float* S_g = state + (size_t)slot[r0] * state_stride + (size_t)h * D * V;
  float S[RPT];
#pragma unroll
  for (int i = 0; i < RPT; ++i) {
    const int d = sub * RPT + i;
    S[i] = (live && d < D) ? S_g[(size_t)d * V + col] : 0.f;
  }
  const int c0 = blockIdx.x * COLS, nc = min(COLS, V - c0);
  const float* q_h = q + (size_t)kh * D;
  const float* k_h = k + (size_t)kh * D;
  const float* g_h = DELTA ? decay + (size_t)h * D : nullptr;
  const float* v_h = v + (size_t)h * V + c0;
  auto fetch = [&](int t0, int st) {
    const int n = min(TB, r1 - t0);
    float* base = stage[st];
    if (VEC) {
      // piece j of a token: 16 bytes of q, then of k, then of the decay, then of the values
      const int d4 = D >> 2, pieces = NV * d4 + (nc >> 2);
      for (int j = tid; j < pieces; j += SCAN_THREADS) {
        int a = 0, x = j;                        // which vector, which piece of it
        if (x >= d4) { x -= d4; a = 1; }
        if (a == 1 && x >= d4) { x -= d4; a = 2; }
        if (DELTA && a == 2 && x >= d4) { x -= d4; a = 3; }
        const bool val = a == NV;
        const int d = 4 * x;
        const int off = val ? NV * DP + d : a * DP + (d / RPT) * SEG + d % RPT;
        const float* src = val ? v_h + d : (a == 0 ? q_h : a == 1 ? k_h : g_h) + d;
        const long long stride = val ? v_stride : a == 0 ? q_stride : a == 1 ? k_stride : (long long)H * D;
        for (int tt = 0; tt < n; ++tt) copy16(base + (size_t)tt * per_tok + off, src + (size_t)(t0 + tt) * stride);
      }
    } else {
      for (int i = tid; i < n * D; i += SCAN_THREADS) {
        const int tt = i / D, d = i % D, t = t0 + tt;
        float* dst = base + (size_t)tt * per_tok + (d / RPT) * SEG + d % RPT;
        copy4(dst, q_h + (size_t)t * q_stride + d);
        copy4(dst + DP, k_h + (size_t)t * k_stride + d);
        if (DELTA) copy4(dst + 2 * DP, g_h + (size_t)t * H * D + d);
      }
      for (int i = tid; i < n * nc; i += SCAN_THREADS) {
        const int tt = i / nc, c = i % nc;
        copy4(base + (size_t)tt * per_tok + NV * DP + c, v_h + (size_t)(t0 + tt) * v_stride + c);
      }
    }
    for (int tt = tid; tt < n; tt += SCAN_THREADS) {
      float* dst = base + (size_t)tt * per_tok + NV * DP + COLS;
      copy4(dst, w1 + (size_t)(t0 + tt) * H + h);
      if (!DELTA) copy4(dst + 1, decay + (size_t)(t0 + tt) * H + h);
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  const float skip_h = skip ? skip[h] : 0.f;
  fetch(r0, 0);
  int st = 0;
  for (int t0 = r0; t0 < r1; t0 += TB, st ^= 1) {
    if (t0 + TB < r1) {
      fetch(t0 + TB, st ^ 1);
      asm volatile("cp.async.wait_group 1;" ::: "memory");
    } else {
      asm volatile("cp.async.wait_group 0;" ::: "memory");
    }
    __syncthreads();
    const int n = min(TB, r1 - t0);
    for (int tt = 0; tt < n; ++tt) {
      const float* tok = stage[st] + (size_t)tt * per_tok;
      const float4* q4 = reinterpret_cast<const float4*>(tok + sub * SEG);
      const float4* k4 = reinterpret_cast<const float4*>(tok + DP + sub * SEG);
      const float* rest = tok + NV * DP;
      const float vj = rest[tid / TPC], w = rest[COLS];
      float4 kr[RPT / 4];                        // the key's dims of this lane, read once for both passes
#pragma unroll
      for (int i = 0; i < RPT / 4; ++i) kr[i] = k4[i];
      float u;
      if (DELTA) {
        const float4* g4 = reinterpret_cast<const float4*>(tok + 2 * DP + sub * SEG);
        float d0 = 0.f, d1 = 0.f, d2 = 0.f, d3 = 0.f;
#pragma unroll
        for (int i = 0; i < RPT / 4; ++i) {
          const float4 gg = g4[i];
          S[4 * i] *= gg.x; S[4 * i + 1] *= gg.y; S[4 * i + 2] *= gg.z; S[4 * i + 3] *= gg.w;
          d0 = fmaf(S[4 * i], kr[i].x, d0); d1 = fmaf(S[4 * i + 1], kr[i].y, d1);
          d2 = fmaf(S[4 * i + 2], kr[i].z, d2); d3 = fmaf(S[4 * i + 3], kr[i].w, d3);
        }
        float dot = (d0 + d1) + (d2 + d3);
#pragma unroll
        for (int m = 1; m < TPC; m <<= 1) dot += __shfl_xor_sync(0xffffffffu, dot, m);
        u = w * (vj - dot);
      } else {
        const float a = rest[COLS + 1];
#pragma unroll
        for (int i = 0; i < RPT; ++i) S[i] *= a;
        u = w * vj;
      }
      float o0 = 0.f, o1 = 0.f, o2 = 0.f, o3 = 0.f;
#pragma unroll
      for (int i = 0; i < RPT / 4; ++i) {
        const float4 qq = q4[i];
        S[4 * i] = fmaf(kr[i].x, u, S[4 * i]); S[4 * i + 1] = fmaf(kr[i].y, u, S[4 * i + 1]);
        S[4 * i + 2] = fmaf(kr[i].z, u, S[4 * i + 2]); S[4 * i + 3] = fmaf(kr[i].w, u, S[4 * i + 3]);
        o0 = fmaf(S[4 * i], qq.x, o0); o1 = fmaf(S[4 * i + 1], qq.y, o1);
        o2 = fmaf(S[4 * i + 2], qq.z, o2); o3 = fmaf(S[4 * i + 3], qq.w, o3);
      }
      float out = (o0 + o1) + (o2 + o3);
#pragma unroll
      for (int m = 1; m < TPC; m <<= 1) out += __shfl_xor_sync(0xffffffffu, out, m);
      if (live && sub == 0) o[(size_t)(t0 + tt) * H * V + (size_t)h * V + col] = fmaf(skip_h, vj, out);
    }
    __syncthreads();          // the stage is refilled in the next round
  }
  // Only now may the kernel behind this one start: its blocks would wait on the SMs beside the walk's few warps for
  // as long as the walk takes (a prompt of 2,048 tokens ran twice as long with the release at the top).
  pdl_launch();
#pragma unroll
  for (int i = 0; i < RPT; ++i) {
    const int d = sub * RPT + i;
    if (live && d < D) S_g[(size_t)d * V + col] = S[i];
  }
}

// ------------------------------------------------------------------------------------------- norm and gate of the heads' outputs
// out = norm(o [* act(gate)]) * w [* act(gate)]: every row's N numbers are divided, in `groups` equal parts, each by its
// own root mean square; w has `w_len` numbers and repeats over the row (a scale per head dim shared by all heads, or
// one per channel).  gate_first: the gate multiplies before the norm, else after.  gate_act: 0 sigmoid, 1 silu.
// One block per (row, group).
template <typename TO>
__global__ void gated_norm_kernel(const float* __restrict__ o, const float* __restrict__ gate, long long gate_stride,
                                  int gate_act, int gate_first, const float* __restrict__ w, int w_len, float eps,
                                  int groups, int N, TO* __restrict__ out) {
  __shared__ float red[32];
  pdl_launch();
  pdl_wait();
  const int t = blockIdx.x / groups, grp = blockIdx.x % groups, gs = N / groups, c0 = grp * gs;
  const float* orow = o + (size_t)t * N + c0;
  const float* grow = gate + (size_t)t * gate_stride + c0;
  float ss = 0.f;
  for (int c = threadIdx.x; c < gs; c += blockDim.x) {
    float x = orow[c];
    if (gate_first) x *= gate_act ? siluf_(grow[c]) : sigmoidf_(grow[c]);
    ss = fmaf(x, x, ss);
  }
  ss = block_sum(ss, red);
  const float inv = 1.0f / sqrtf(ss / (float)gs + eps);
  for (int c = threadIdx.x; c < gs; c += blockDim.x) {
    const float gt = gate_act ? siluf_(grow[c]) : sigmoidf_(grow[c]);
    float x = orow[c];
    if (gate_first) x = x * gt * inv * w[(c0 + c) % w_len];
    else x = x * inv * w[(c0 + c) % w_len] * gt;
    out[(size_t)t * N + c0 + c] = from_f32<TO>(x);
  }
}

// ------------------------------------------------------------------------------------------- weighted sums of branches, normed, added
struct SumList {
  const float* partials[4];
  long long stride[4];       // between partial sums
  int n_partials[4];
  const float* bias[4];
  float scale[4];
  int n;
  const float* y;            // rows of chosen experts [*, W] (or null), the places of a token's rows and their weights
  const int* row_of;
  const float* gates;
  int k;
};

// r[t] = sum_b scale_b * y_b[t] + sum_j gates[t, j] * y[row_of[t, j]], y_b the sum of branch b's partial sums (+ bias);
// with gamma: r <- r / sqrt(mean(r^2) + eps) * gamma; then dst[t] += r (accumulate) or dst[t] = r.
__global__ void sum_norm_add_kernel(SumList sl, const float* __restrict__ gamma, float eps, float* __restrict__ dst,
                                    int accumulate, int W) {
  __shared__ float red[32];
  pdl_launch();
  pdl_wait();
  const int t = blockIdx.x;
  auto value = [&](int c) {
    float r = 0.f;
    for (int b = 0; b < sl.n; ++b) {
      float x = 0.f;
      for (int z = 0; z < sl.n_partials[b]; ++z) x += sl.partials[b][(size_t)z * sl.stride[b] + (size_t)t * W + c];
      if (sl.bias[b]) x += sl.bias[b][c];
      r = fmaf(sl.scale[b], x, r);
    }
    for (int j = 0; j < sl.k; ++j)
      r = fmaf(sl.gates[(size_t)t * sl.k + j], sl.y[(size_t)sl.row_of[(size_t)t * sl.k + j] * W + c], r);
    return r;
  };
  float inv = 1.f;
  if (gamma) {
    float ss = 0.f;
    for (int c = threadIdx.x; c < W; c += blockDim.x) {
      const float x = value(c);
      ss = fmaf(x, x, ss);
    }
    ss = block_sum(ss, red);
    inv = 1.0f / sqrtf(ss / (float)W + eps);
  }
  for (int c = threadIdx.x; c < W; c += blockDim.x) {
    float r = value(c) * inv;
    if (gamma) r *= gamma[c];
    float* d = dst + (size_t)t * W + c;
    *d = accumulate ? *d + r : r;
  }
}

// The same with rows of whole 16-byte units, every pointer on 16 bytes: a thread holds up to four units of the row in
// registers between the sum of squares and the store, so the row's operands are read once and the blocks are small
// enough that several share an SM.
__global__ void sum_norm_add_vec_kernel(SumList sl, const float* __restrict__ gamma, float eps, float* __restrict__ dst,
                                        int accumulate, int W) {
  __shared__ float red[32];
  pdl_launch();
  pdl_wait();
  constexpr int U = 4;
  const int t = blockIdx.x, n4 = W / 4;
  float4 v[U];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < U; ++i) {
    const int c4 = threadIdx.x + i * blockDim.x;
    float4 r = make_float4(0.f, 0.f, 0.f, 0.f);
    if (c4 < n4) {
      for (int b = 0; b < sl.n; ++b) {
        float4 x = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int z = 0; z < sl.n_partials[b]; ++z) {
          const float4 q = *reinterpret_cast<const float4*>(sl.partials[b] + (size_t)z * sl.stride[b] + (size_t)t * W + 4 * c4);
          x.x += q.x; x.y += q.y; x.z += q.z; x.w += q.w;
        }
        if (sl.bias[b]) {
          const float4 q = *reinterpret_cast<const float4*>(sl.bias[b] + 4 * c4);
          x.x += q.x; x.y += q.y; x.z += q.z; x.w += q.w;
        }
        const float sc = sl.scale[b];
        r.x = fmaf(sc, x.x, r.x); r.y = fmaf(sc, x.y, r.y); r.z = fmaf(sc, x.z, r.z); r.w = fmaf(sc, x.w, r.w);
      }
      for (int j = 0; j < sl.k; ++j) {
        const float gt = sl.gates[(size_t)t * sl.k + j];
        const float4 q = *reinterpret_cast<const float4*>(sl.y + (size_t)sl.row_of[(size_t)t * sl.k + j] * W + 4 * c4);
        r.x = fmaf(gt, q.x, r.x); r.y = fmaf(gt, q.y, r.y); r.z = fmaf(gt, q.z, r.z); r.w = fmaf(gt, q.w, r.w);
      }
    }
    v[i] = r;
    ss = fmaf(r.x, r.x, fmaf(r.y, r.y, fmaf(r.z, r.z, fmaf(r.w, r.w, ss))));
  }
  float inv = 1.f;
  if (gamma) {
    ss = block_sum(ss, red);
    inv = 1.0f / sqrtf(ss / (float)W + eps);
  }
#pragma unroll
  for (int i = 0; i < U; ++i) {
    const int c4 = threadIdx.x + i * blockDim.x;
    if (c4 >= n4) continue;
    float4 r = v[i];
    if (gamma) {
      const float4 gm = *reinterpret_cast<const float4*>(gamma + 4 * c4);
      r.x *= inv * gm.x; r.y *= inv * gm.y; r.z *= inv * gm.z; r.w *= inv * gm.w;
    }
    float4* d = reinterpret_cast<float4*>(dst + (size_t)t * W + 4 * c4);
    if (accumulate) {
      const float4 o = *d;
      r.x += o.x; r.y += o.y; r.z += o.z; r.w += o.w;
    }
    *d = r;
  }
}

// ------------------------------------------------------------------------------------------- retention: rotated q and k, constant decays
// proj [T, >= 2 H D] float32 (q | k of H heads of D dims): the leading `rot` dims of every head turn by the row's
// position into qk [T, 2 H D]; decay [T, H] gets the head's fixed decay and dt [T, H] the constant that scales what is
// written into the state (the recurrence kernel takes both per token).
__global__ void retention_prepare_kernel(const float* __restrict__ proj, long long stride, const int* __restrict__ pos,
                                         const float* __restrict__ cos_t, const float* __restrict__ sin_t, int rot,
                                         int interleaved, const float* __restrict__ decay_h, float dt_value,
                                         float* __restrict__ qk, float* __restrict__ decay, float* __restrict__ dt, int H,
                                         int D) {
  pdl_launch();
  pdl_wait();
  const int t = blockIdx.x, p = pos[t], half = rot / 2, n = 2 * H * D;
  const float* row = proj + (size_t)t * stride;
  for (int e = threadIdx.x; e < n; e += blockDim.x) {
    const int d = e % D;
    float x = row[e];
    if (d < rot) {
      int i, partner;
      bool first;
      if (interleaved) { i = d >> 1; first = !(d & 1); partner = first ? e + 1 : e - 1; }
      else { i = d < half ? d : d - half; first = d < half; partner = first ? e + half : e - half; }
      const float z = row[partner];
      const float c = cos_t[(size_t)p * half + i], s = sin_t[(size_t)p * half + i];
      x = first ? x * c - z * s : x * c + z * s;
    }
    qk[(size_t)t * n + e] = x;
  }
  for (int h = threadIdx.x; h < H; h += blockDim.x) {
    decay[(size_t)t * H + h] = decay_h[h];
    dt[(size_t)t * H + h] = dt_value;
  }
}

// ------------------------------------------------------------------------------------------- mean of normed branches
struct BranchList {
  const float* partials[4];
  long long stride[4];       // between partial sums
  int n_partials[4];
  const float* bias[4];
  const float* w[4];
  int n;
};

// out[t] = (1 / n) sum_b w_b * y_b / sqrt(mean(y_b^2) + eps), y_b = the sum of branch b's partial sums (+ bias).
__global__ void branch_mean_kernel(BranchList bl, float eps, float* __restrict__ out, int W) {
  __shared__ float red[32];
  pdl_launch();
  pdl_wait();
  const int t = blockIdx.x;
  float inv[4];
  auto value = [&](int b, int c) {
    float x = 0.f;
    for (int z = 0; z < bl.n_partials[b]; ++z) x += bl.partials[b][(size_t)z * bl.stride[b] + (size_t)t * W + c];
    return bl.bias[b] ? x + bl.bias[b][c] : x;
  };
  for (int b = 0; b < bl.n; ++b) {
    float ss = 0.f;
    for (int c = threadIdx.x; c < W; c += blockDim.x) {
      const float x = value(b, c);
      ss = fmaf(x, x, ss);
    }
    ss = block_sum(ss, red);
    inv[b] = 1.0f / sqrtf(ss / (float)W + eps);
  }
  const float share = 1.0f / (float)bl.n;
  for (int c = threadIdx.x; c < W; c += blockDim.x) {
    float acc = 0.f;
    for (int b = 0; b < bl.n; ++b) acc = fmaf(value(b, c) * inv[b], bl.w[b][c], acc);
    out[(size_t)t * W + c] = acc * share;
  }
}

// ------------------------------------------------------------------------------------------- norm after the sum
// x[t] <- norm(a x[t] + s * (sum of partial sums + bias)) in place, s [W] or null (ones); mode 0 LayerNorm (the
// variance is the mean of the squared deviations), 1 RMSNorm; `copy` receives the result in another type too.  The
// row waits in shared memory between the passes.  One block per row.
template <typename TC>
__global__ void post_norm_kernel(float* __restrict__ x, const float* __restrict__ partials, int n_partials,
                                 long long partial_stride, const float* __restrict__ bias, const float* __restrict__ s,
                                 float a, const float* __restrict__ gamma, const float* __restrict__ beta, float eps,
                                 int mode, TC* __restrict__ copy, int W) {
  extern __shared__ float rowbuf[];
  __shared__ float red[32];
  pdl_launch();
  pdl_wait();
  const int t = blockIdx.x;
  float sum = 0.f;
  for (int c = threadIdx.x; c < W; c += blockDim.x) {
    float y = 0.f;
    for (int z = 0; z < n_partials; ++z) y += partials[(size_t)z * partial_stride + (size_t)t * W + c];
    if (bias) y += bias[c];
    if (s) y *= s[c];
    const float v = fmaf(a, x[(size_t)t * W + c], y);
    rowbuf[c] = v;
    sum += v;
  }
  float mean = 0.f;
  if (mode == 0) mean = block_sum(sum, red) / (float)W;
  float ss = 0.f;
  for (int c = threadIdx.x; c < W; c += blockDim.x) {
    const float d = rowbuf[c] - mean;
    ss = fmaf(d, d, ss);
  }
  ss = block_sum(ss, red);
  const float inv = 1.0f / sqrtf(ss / (float)W + eps);
  for (int c = threadIdx.x; c < W; c += blockDim.x) {
    float v = (rowbuf[c] - mean) * inv * gamma[c];
    if (beta) v += beta[c];
    x[(size_t)t * W + c] = v;
    if (copy) copy[(size_t)t * W + c] = from_f32<TC>(v);
  }
}

// ------------------------------------------------------------------------------------------- weighted sum over depth
// hist [L, T W]: hist[n - 1] <- h, then h <- sum_{j < n} w[j] hist[j] (ascending j), and a copy in another type.
template <typename TC>
__global__ void depth_mix_kernel(float* __restrict__ hist, long long level_stride, int n, const float* __restrict__ w,
                                 float* __restrict__ h, TC* __restrict__ copy, long long count) {
  pdl_launch();
  pdl_wait();
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= count) return;
  const float cur = h[i];
  hist[(size_t)(n - 1) * level_stride + i] = cur;
  float acc = 0.f;
  for (int j = 0; j < n - 1; ++j) acc = fmaf(w[j], hist[(size_t)j * level_stride + i], acc);
  acc = fmaf(w[n - 1], cur, acc);
  h[i] = acc;
  if (copy) copy[i] = from_f32<TC>(acc);
}

__global__ void softcap_kernel(float* __restrict__ x, float cap, long long count) {
  pdl_launch();
  pdl_wait();
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < count) x[i] = cap * tanhf(x[i] / cap);
}

template <typename TC>
__global__ void cast_rows_kernel(const float* __restrict__ x, TC* __restrict__ out, long long count) {
  pdl_launch();
  pdl_wait();
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < count) out[i] = from_f32<TC>(x[i]);
}

// ------------------------------------------------------------------------------------------- q, k, v on their way to the cache
// y [T, (nq + nkv) hd + nkv vd] float32: q | k | v.  Every q and k head is divided by its root mean square (eps) and
// scaled by qw / kw [hd] (null: no norm), then its leading `rot` dims rotate by the row's position; every v head's
// vd dims rotate by the row's position with tables of their own (null: as they are).  q goes to q_out, k and v into
// the row's cache page.  One block per row, a warp per head.
template <typename TQ, typename TC>
__global__ void qk_norm_write_kernel(const float* __restrict__ y, long long y_stride, const float* __restrict__ qw,
                                     const float* __restrict__ kw, float eps, const int* __restrict__ pos,
                                     const int* __restrict__ slot, const float* __restrict__ cos_t,
                                     const float* __restrict__ sin_t, int rot, int interleaved,
                                     const float* __restrict__ vcos, const float* __restrict__ vsin, int v_interleaved,
                                     TQ* __restrict__ q_out, TC* __restrict__ k_cache, TC* __restrict__ v_cache,
                                     const int* __restrict__ block_table, int max_pages, int page_size, int nq, int nkv,
                                     int hd, int vd, int whole, int v_from_k, float qt_coef, int qt_every,
                                     int* __restrict__ status) {
  __shared__ float part[2][32];
  pdl_launch();
  pdl_wait();
  const int t = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  const int p = pos[t], lp = p / page_size;
  const int page = lp < max_pages ? block_table[(size_t)slot[t] * max_pages + lp] : -1;
  if (page < 0 && threadIdx.x == 0) atomicExch(status, 1);
  const float* row = y + (size_t)t * y_stride;
  // a temperature on the queries that grows with the position: 1 + coef ln(floor((p + 1) / every) + 1)
  const float q_temp = qt_coef != 0.f ? 1.0f + qt_coef * logf(floorf((float)(p + 1) / (float)qt_every) + 1.0f) : 1.0f;
  float inv_whole[2] = {1.f, 1.f};
  if (whole && qw) {          // one root mean square over all query heads, one over all key heads
    float sq = 0.f, sk = 0.f;
    for (int e = threadIdx.x; e < nq * hd; e += blockDim.x) sq = fmaf(row[e], row[e], sq);
    for (int e = threadIdx.x; e < nkv * hd; e += blockDim.x) sk = fmaf(row[(size_t)nq * hd + e], row[(size_t)nq * hd + e], sk);
    sq = warp_sum(sq);
    sk = warp_sum(sk);
    if (lane == 0) { part[0][warp] = sq; part[1][warp] = sk; }
    __syncthreads();
    sq = sk = 0.f;
    for (int i = 0; i < nw; ++i) { sq += part[0][i]; sk += part[1][i]; }      // the same order in every thread
    inv_whole[0] = 1.0f / sqrtf(sq / (float)(nq * hd) + eps);
    inv_whole[1] = 1.0f / sqrtf(sk / (float)(nkv * hd) + eps);
  }
  for (int head = warp; head < nq + 2 * nkv; head += nw) {
    const bool is_v = head >= nq + nkv;
    const int n = is_v ? vd : hd;
    // values that are the keys as projected come from the key's columns (vd = hd), before norm and rotation
    const float* src = is_v ? (v_from_k ? row + (size_t)(head - nkv) * hd
                                        : row + (size_t)(nq + nkv) * hd + (size_t)(head - nq - nkv) * vd)
                            : row + (size_t)head * hd;
    const float* w = is_v ? nullptr : (head < nq ? qw : kw);
    float inv = 1.f;
    if (w && whole) {
      inv = inv_whole[head < nq ? 0 : 1];
      w += (size_t)(head < nq ? head : head - nq) * hd;       // a scale per column of the projection
    } else if (w) {
      float ss = 0.f;
      for (int d = lane; d < n; d += 32) ss = fmaf(src[d], src[d], ss);
      inv = 1.0f / sqrtf(warp_sum(ss) / (float)n + eps);
    }
    if (head < nq) inv *= q_temp;
    const float* ct = is_v ? vcos : cos_t;
    const float* st = is_v ? vsin : sin_t;
    const int r = is_v ? (vcos ? vd : 0) : rot, half = r / 2, il = is_v ? v_interleaved : interleaved;
    for (int d = lane; d < n; d += 32) {
      float x = src[d] * inv * (w ? w[d] : 1.f);
      if (d < r) {
        int i, partner;
        bool first;
        if (il) { i = d >> 1; first = !(d & 1); partner = first ? d + 1 : d - 1; }
        else { i = d < half ? d : d - half; first = d < half; partner = first ? d + half : d - half; }
        const float z = src[partner] * inv * (w ? w[partner] : 1.f);
        const float c = ct[(size_t)p * half + i], s = st[(size_t)p * half + i];
        x = first ? x * c - z * s : x * c + z * s;
      }
      if (head < nq) {
        q_out[((size_t)t * nq + head) * hd + d] = from_f32<TQ>(x);
      } else if (page >= 0) {
        if (!is_v) k_cache[(((size_t)page * nkv + (head - nq)) * page_size + p % page_size) * hd + d] = from_f32<TC>(x);
        else v_cache[(((size_t)page * nkv + (head - nq - nkv)) * page_size + p % page_size) * vd + d] = from_f32<TC>(x);
      }
    }
  }
}

// attn [T, nq vd]: every head's sum is rotated back by the row's position (tables null: not at all) and multiplied by
// sigmoid(gate[t, head]) (gate null: by 1).  One thread per pair of dims.
template <typename TA>
__global__ void head_finish_kernel(const TA* __restrict__ attn, const int* __restrict__ pos, const float* __restrict__ vcos,
                                   const float* __restrict__ vsin, int interleaved, const float* __restrict__ gate,
                                   long long gate_stride, int gate_each, TA* __restrict__ out, int T, int nq, int vd) {
  pdl_launch();
  pdl_wait();
  const int half = vd / 2;
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (long long)T * nq * half) return;
  const int i = (int)(idx % half), head = (int)((idx / half) % nq), t = (int)(idx / ((long long)half * nq));
  const int a = interleaved ? 2 * i : i, b = interleaved ? 2 * i + 1 : i + half;
  const size_t base = ((size_t)t * nq + head) * vd;
  float u = to_f32(attn[base + a]), v = to_f32(attn[base + b]);
  if (vcos) {
    const float c = vcos[(size_t)pos[t] * half + i], s = vsin[(size_t)pos[t] * half + i];
    const float u2 = u * c + v * s, v2 = v * c - u * s;       // the angle's sign turned round
    u = u2;
    v = v2;
  }
  // a gate per head, or one per number of every head
  const float* gr = gate + (size_t)t * gate_stride;
  const float ga = !gate ? 1.f : sigmoidf_(gate_each ? gr[(size_t)head * vd + a] : gr[head]);
  const float gb = !gate ? 1.f : (gate_each ? sigmoidf_(gr[(size_t)head * vd + b]) : ga);
  out[base + a] = from_f32<TA>(u * ga);
  out[base + b] = from_f32<TA>(v * gb);
}

}  // namespace

// =========================================================================================== launchers
// Threads of a block that takes a whole row of W numbers, each summed from several partial sums: two numbers a thread,
// so that a batch of a few rows still has many loads in flight.
static int row_threads(int W) { return W >= 2048 ? 1024 : W >= 1024 ? 512 : W >= 512 ? 256 : 128; }

extern "C" int flint_short_conv(const float* u, long long in_stride, int col0, const float* w, const float* bias, int act,
                                const int* pos, const int* slot, float* ring, long long ring_stride, float* y, int T,
                                int C, int taps, cudaStream_t stream) {
  if (T <= 0 || C <= 0) return 0;
  if (taps < 1 || taps > 64) return fail("short_conv: %d taps are not supported (1 to 64)", taps);
  if (taps > 1 && !ring) return fail("short_conv: a convolution over time needs the requests' state");
  // few rows (decoded tokens): a thread a channel, so that the rows spread over the chip; many rows: four channels a thread
  const int threads = C >= 1024 ? 256 : 128, per = T >= 256 ? 4 : 1;
  const dim3 grid((unsigned)T, (unsigned)min((C + threads * per - 1) / (threads * per), 65535));
  launch_pdl(short_conv_kernel, grid, dim3(threads), 0, stream, u, in_stride, col0, w, bias, act, pos, slot,
             (const float*)ring, ring_stride, y, T, C, taps);
  if (taps > 1)
    launch_pdl(short_conv_keep_kernel, grid, dim3(threads), 0, stream, u, in_stride, col0, pos, slot, ring, ring_stride, T, C,
               taps);
  return check_launch("short_conv");
}

extern "C" int flint_delta_prepare(const float* y, long long y_stride, const float* b, long long b_stride, const float* a,
                                   const float* dt_bias, const float* a_log, float* qk, float* decay, float* beta, int T,
                                   int H, int G, int D, float unit_eps, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (G <= 0 || H % G) return fail("delta_prepare: %d heads do not divide into %d key heads", H, G);
  launch_pdl(delta_prepare_kernel, dim3((unsigned)T), dim3(256), 0, stream, y, y_stride, b, b_stride, a, dt_bias, a_log, qk,
             decay, beta, H, G, D, unit_eps);
  return check_launch("delta_prepare");
}

extern "C" int flint_ssd_prepare(const float* raw, long long raw_stride, const float* dt_bias, const float* a_log, float* dt,
                                 float* decay, int T, int H, cudaStream_t stream) {
  if (T <= 0) return 0;
  launch_pdl(ssd_prepare_kernel, dim3((unsigned)((T * (long long)H + 127) / 128)), dim3(128), 0, stream, raw, raw_stride,
             dt_bias, a_log, dt, decay, T, H);
  return check_launch("ssd_prepare");
}

template <typename... KArgs, typename... Args>
static cudaError_t launch_scan(bool early, void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                               Args&&... args) {
  if (early) return launch_pdl(kernel, grid, block, smem, stream, static_cast<Args&&>(args)...);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

extern "C" int flint_recurrence_scan(const float* q, long long q_stride, const float* k, long long k_stride, const float* v,
                                     long long v_stride, const float* decay, int delta, const float* w1, const float* skip,
                                     const int* slot, const int* seq_start, int n_seq, float* state,
                                     long long state_stride, float* o, int H, int G, int D, int V, cudaStream_t stream) {
  if (n_seq <= 0) return 0;
  if (D < 1 || D > 256 || V < 1) return fail("recurrence_scan: %d key dims per head are not supported (1 to 256)", D);
  if (G <= 0 || H % G) return fail("recurrence_scan: %d heads do not divide into %d key heads", H, G);
  if (n_seq > 65535 || H > 65535) return fail("recurrence_scan: too many requests or heads");
  const int tpc = D <= 32 ? 1 : D <= 64 ? 2 : D <= 128 ? 4 : 8;
  const int dp = tpc * SEG, cols = SCAN_THREADS / tpc;
  const int tb = tpc <= 2 ? 16 : tpc <= 4 ? 8 : 4;
  const size_t smem = (size_t)2 * tb * ((delta ? 3 : 2) * dp + cols + 4) * sizeof(float);
  const dim3 grid((unsigned)((V + cols - 1) / cols), (unsigned)H, (unsigned)n_seq), block(SCAN_THREADS);
  // 16-byte copies need every staged row to start on such a boundary
  auto lined = [](const void* p) { return ((uintptr_t)p & 15) == 0; };
  const bool vec = D % 4 == 0 && V % 4 == 0 && q_stride % 4 == 0 && k_stride % 4 == 0 && v_stride % 4 == 0 && lined(q) &&
                   lined(k) && lined(v) && (!delta || lined(decay));
  // A walk over prompts starts as an ordinary dependent, on an empty chip, where its few blocks get an SM each: started
  // early they land beside the blocks of the kernel before, several to an SM (a prompt of 2,048 tokens then ran half
  // a millisecond longer a layer).  A batch of single tokens fills the chip anyway and starts early.
  const bool early = seq_start == nullptr;
#define SCAN(TPC, DELTA, VEC)                                                                                          \
  launch_scan(early, recurrence_scan_kernel<TPC, DELTA, VEC>, grid, block, smem, stream, q, q_stride, k, k_stride, v,   \
              v_stride, decay, w1, skip, slot, seq_start, state, state_stride, o, H, G, D, V, tb)
#define SCAN_T(TPC)                                                                                       \
  do {                                                                                                    \
    if (delta) { if (vec) SCAN(TPC, true, true); else SCAN(TPC, true, false); }                           \
    else { if (vec) SCAN(TPC, false, true); else SCAN(TPC, false, false); }                               \
  } while (0)
  if (tpc == 1) SCAN_T(1);
  else if (tpc == 2) SCAN_T(2);
  else if (tpc == 4) SCAN_T(4);
  else SCAN_T(8);
#undef SCAN_T
#undef SCAN
  return check_launch("recurrence_scan");
}

extern "C" int flint_gated_norm(const float* o, const float* gate, long long gate_stride, int gate_act, int gate_first,
                                const float* w, int w_len, float eps, int groups, int N, void* out, int out_dtype, int T,
                                cudaStream_t stream) {
  if (T <= 0) return 0;
  if (groups < 1 || N % groups || w_len < 1) return fail("gated_norm: %d numbers do not divide into %d parts", N, groups);
  if ((long long)T * groups > 0x7fffffffLL) return fail("gated_norm: too many rows");
  const int gs = N / groups, threads = gs >= 1024 ? 256 : gs > 64 ? 128 : gs > 32 ? 64 : 32;
  FLINT_DISPATCH_DTYPE(out_dtype, TO,
      launch_pdl(gated_norm_kernel<TO>, dim3((unsigned)(T * groups)), dim3(threads), 0, stream, o, gate, gate_stride, gate_act,
                 gate_first, w, w_len, eps, groups, N, (TO*)out));
  return check_launch("gated_norm");
}

extern "C" int flint_sum_norm_add(int n, const float* const* partials, const long long* strides, const int* n_partials,
                                  const float* const* bias, const float* scales, const float* y, const int* row_of,
                                  const float* gates, int k, const float* gamma, float eps, float* dst, int accumulate,
                                  int T, int W, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (n < 0 || n > 4) return fail("sum_norm_add: %d branches are not supported (up to 4)", n);
  if (k < 0 || (k > 0 && (!y || !row_of || !gates))) return fail("sum_norm_add: expert rows need their places and weights");
  if (n == 0 && k == 0) return fail("sum_norm_add: nothing to add");
  SumList sl = {};
  sl.n = n;
  for (int b = 0; b < n; ++b) {
    sl.partials[b] = partials[b];
    sl.stride[b] = strides[b];
    sl.n_partials[b] = n_partials[b];
    sl.bias[b] = bias[b];
    sl.scale[b] = scales[b];
  }
  sl.y = y; sl.row_of = row_of; sl.gates = gates; sl.k = k;
  bool vec = W % 4 == 0 && W <= 4 * 4 * 1024 && !(((uintptr_t)dst | (uintptr_t)gamma | (uintptr_t)y) & 15);
  for (int b = 0; b < n && vec; ++b)
    vec = !(((uintptr_t)partials[b] | (uintptr_t)bias[b]) & 15) && strides[b] % 4 == 0;
  if (vec) {
    int threads = ((W / 16 + 31) / 32) * 32;          // four 16-byte units a thread
    if (threads < 64) threads = 64;
    launch_pdl(sum_norm_add_vec_kernel, dim3((unsigned)T), dim3(threads), 0, stream, sl, gamma, eps, dst, accumulate, W);
  } else {
    launch_pdl(sum_norm_add_kernel, dim3((unsigned)T), dim3(row_threads(W)), 0, stream, sl, gamma, eps, dst, accumulate, W);
  }
  return check_launch("sum_norm_add");
}

extern "C" int flint_retention_prepare(const float* proj, long long stride, const int* pos, const float* cos_t,
                                       const float* sin_t, int rot, int interleaved, const float* decay_h, float dt_value,
                                       float* qk, float* decay, float* dt, int T, int H, int D, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (rot < 0 || rot > D || rot % 2) return fail("retention_prepare: %d rotating dims do not fit heads of %d", rot, D);
  launch_pdl(retention_prepare_kernel, dim3((unsigned)T), dim3(2 * H * D >= 1024 ? 256 : 128), 0, stream, proj, stride, pos,
             cos_t, sin_t, rot, interleaved, decay_h, dt_value, qk, decay, dt, H, D);
  return check_launch("retention_prepare");
}

extern "C" int flint_branch_mean(int n, const float* const* partials, const long long* strides, const int* n_partials,
                                 const float* const* bias, const float* const* w, float eps, float* out, int T, int W,
                                 cudaStream_t stream) {
  if (T <= 0) return 0;
  if (n < 1 || n > 4) return fail("branch_mean: %d branches are not supported (1 to 4)", n);
  BranchList bl = {};
  bl.n = n;
  for (int b = 0; b < n; ++b) {
    bl.partials[b] = partials[b];
    bl.stride[b] = strides[b];
    bl.n_partials[b] = n_partials[b];
    bl.bias[b] = bias[b];
    bl.w[b] = w[b];
  }
  launch_pdl(branch_mean_kernel, dim3((unsigned)T), dim3(row_threads(W)), 0, stream, bl, eps, out, W);
  return check_launch("branch_mean");
}

extern "C" int flint_post_norm(float* x, const float* partials, int n_partials, long long partial_stride, const float* bias,
                               const float* s, float a, const float* gamma, const float* beta, float eps, int mode,
                               void* copy, int copy_dtype, int T, int W, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (n_partials < 1) return fail("post_norm: needs at least one partial sum");
  const size_t smem = (size_t)W * sizeof(float);
  if (smem > 200 * 1024) return fail("post_norm: rows of %d numbers are not supported", W);
  if (smem > 48 * 1024) {
    cudaFuncSetAttribute(post_norm_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    cudaFuncSetAttribute(post_norm_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
  }
  FLINT_DISPATCH_DTYPE(copy_dtype, TC,
      launch_pdl(post_norm_kernel<TC>, dim3((unsigned)T), dim3(row_threads(W)), smem, stream, x, partials, n_partials,
                 partial_stride, bias, s, a, gamma, beta, eps, mode, (TC*)copy, W));
  return check_launch("post_norm");
}

extern "C" int flint_depth_mix(float* hist, long long level_stride, int n, const float* w, float* h, void* copy,
                               int copy_dtype, long long count, cudaStream_t stream) {
  if (count <= 0) return 0;
  if (n < 1) return fail("depth_mix: needs at least one level");
  FLINT_DISPATCH_DTYPE(copy_dtype, TC,
      launch_pdl(depth_mix_kernel<TC>, dim3((unsigned)((count + 255) / 256)), dim3(256), 0, stream, hist, level_stride, n, w,
                 h, (TC*)copy, count));
  return check_launch("depth_mix");
}

extern "C" int flint_softcap(float* x, float cap, long long count, cudaStream_t stream) {
  if (count <= 0) return 0;
  if (!(cap > 0.f)) return fail("softcap: the cap must be positive");
  launch_pdl(softcap_kernel, dim3((unsigned)((count + 255) / 256)), dim3(256), 0, stream, x, cap, count);
  return check_launch("softcap");
}

extern "C" int flint_cast_rows(const float* x, void* out, int out_dtype, long long count, cudaStream_t stream) {
  if (count <= 0) return 0;
  FLINT_DISPATCH_DTYPE(out_dtype, TC,
      launch_pdl(cast_rows_kernel<TC>, dim3((unsigned)((count + 255) / 256)), dim3(256), 0, stream, x, (TC*)out, count));
  return check_launch("cast_rows");
}

extern "C" int flint_qk_norm_write(const float* y, long long y_stride, const float* qw, const float* kw, float eps,
                                   const int* pos, const int* slot, const float* cos_t, const float* sin_t, int rot,
                                   int interleaved, const float* vcos, const float* vsin, int v_interleaved, void* q_out,
                                   int q_dtype, void* k_cache, void* v_cache, int cache_dtype, const int* block_table,
                                   int max_pages, int page_size, int T, int nq, int nkv, int hd, int vd, int whole, int v_from_k,
                                   float qt_coef, int qt_every, int* status, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (rot < 0 || rot > hd || rot % 2 || (vcos && vd % 2)) return fail("qk_norm_write: bad rotation sizes");
  if (v_from_k && vd != hd) return fail("qk_norm_write: values that are the keys need vd = hd");
  if (qt_coef != 0.f && qt_every < 1) return fail("qk_norm_write: the query temperature's period must be positive");
  if ((qw == nullptr) != (kw == nullptr)) return fail("qk_norm_write: q and k are normed together or not at all");
  FLINT_DISPATCH_DTYPE(q_dtype, TQ, FLINT_DISPATCH_DTYPE(cache_dtype, TC,
      launch_pdl(qk_norm_write_kernel<TQ, TC>, dim3((unsigned)T), dim3(256), 0, stream, y, y_stride, qw, kw, eps, pos, slot,
                 cos_t, sin_t, rot, interleaved, vcos, vsin, v_interleaved, (TQ*)q_out, (TC*)k_cache, (TC*)v_cache,
                 block_table, max_pages, page_size, nq, nkv, hd, vd, whole, v_from_k, qt_coef, qt_every, status)));
  return check_launch("qk_norm_write");
}

extern "C" int flint_head_finish(const void* attn, int dtype, const int* pos, const float* vcos, const float* vsin,
                                 int interleaved, const float* gate, long long gate_stride, int gate_each, void* out, int T,
                                 int nq, int vd, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (vd % 2) return fail("head_finish: value heads of %d dims cannot rotate in pairs", vd);
  const long long n = (long long)T * nq * (vd / 2);
  FLINT_DISPATCH_DTYPE(dtype, TA,
      launch_pdl(head_finish_kernel<TA>, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, stream, (const TA*)attn, pos, vcos,
                 vsin, interleaved, gate, gate_stride, gate_each, (TA*)out, T, nq, vd));
  return check_launch("head_finish");
}

extern "C" const char* flint_recurrent_last_error() { return g_error; }
