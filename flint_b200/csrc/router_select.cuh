// The choice of a softmax router limited to groups, by one warp, from float32 logits in shared memory.
//
//   s = softmax(logits); the E experts form n_groups equal groups of neighbours; a group scores as its best member;
//   only members of the `keep` best groups may be chosen; the `top` best of those are (the lower index among
//   equals); gates: s_e / (sum of the chosen s + 1e-20) * out_scale.
//
// Shared by the stand-alone router kernel (moe.cu) and the row kernel that routes while it has the normalised row
// (row_fused.cu).  `s` holds the logits on entry and the scores afterwards; all 32 lanes of the warp call.
#pragma once
#include <math.h>
#include "common.cuh"

namespace flint {

constexpr int ROUTER_MAX_E = 256;       // experts at most
constexpr int ROUTER_MAX_TOP = 16;      // choices a token at most

__device__ __forceinline__ void select_topk_by_warp(float* s, int lane, int E, int top, int n_groups, int keep,
                                                    float out_scale, int* ids, float* gates) {
  constexpr int EPL = ROUTER_MAX_E / 32;   // lane l holds experts l, l + 32, ...
  float v[EPL];
  float m = -INFINITY;
#pragma unroll
  for (int i = 0; i < EPL; ++i) {
    const int e = lane + 32 * i;
    v[i] = e < E ? s[e] : -INFINITY;
    m = fmaxf(m, v[i]);
  }
  m = warp_max(m);
  float denom = 0.f;
#pragma unroll
  for (int i = 0; i < EPL; ++i) {
    v[i] = lane + 32 * i < E ? expf(v[i] - m) : 0.f;
    denom += v[i];
  }
  denom = warp_sum(denom);
  __syncwarp();
#pragma unroll
  for (int i = 0; i < EPL; ++i) {
    const int e = lane + 32 * i;
    v[i] = e < E ? v[i] / denom : -1.f;          // scores; -1 marks what cannot be chosen
    if (e < E) s[e] = v[i];
  }
  __syncwarp();
  // the best of (value, index) pairs over the warp: the larger value, the lower index among equals
  auto best_of_warp = [&](float& val, int& idx) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, val, o);
      const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
      if (ov > val || (ov == val && oi < idx)) { val = ov; idx = oi; }
    }
  };
  const int per = E / n_groups;
  if (keep < n_groups) {
    float gs[2];                                  // the scores of groups lane and lane + 32
#pragma unroll
    for (int k = 0; k < 2; ++k) {
      const int g = lane + 32 * k;
      gs[k] = -1.f;
      if (g < n_groups)
        for (int e = g * per; e < (g + 1) * per; ++e) gs[k] = fmaxf(gs[k], s[e]);
    }
    unsigned long long kept = 0ull;
    for (int r = 0; r < keep; ++r) {
      float val = gs[0];
      int idx = lane;
      if (gs[1] > val) { val = gs[1]; idx = lane + 32; }
      best_of_warp(val, idx);
      kept |= 1ull << idx;
      if ((idx & 31) == lane) gs[idx >> 5] = -2.f;
    }
#pragma unroll
    for (int i = 0; i < EPL; ++i) {
      const int e = lane + 32 * i;
      if (e < E && !((kept >> (e / per)) & 1ull)) v[i] = -1.f;
    }
  }
  float my_val = 0.f, sum = 0.f;
  int my_sel = 0;
  for (int r = 0; r < top; ++r) {
    float val = -1.f;
    int idx = 0x7fffffff;
#pragma unroll
    for (int i = 0; i < EPL; ++i)
      if (v[i] > val) { val = v[i]; idx = lane + 32 * i; }
    best_of_warp(val, idx);
    if ((idx & 31) == lane) {
#pragma unroll
      for (int i = 0; i < EPL; ++i)
        if (i == (idx >> 5)) v[i] = -1.f;
    }
    if (lane == r) { my_val = val; my_sel = idx; }
    sum += val;
  }
  if (lane < top) {
    ids[lane] = my_sel;
    gates[lane] = my_val / (sum + 1e-20f) * out_scale;
  }
}

// The choice of a sigmoid router, by one warp, from float32 logits in shared memory: scores sigmoid(logit) over the
// first E entries, the `top` largest chosen (the lower index among equals), their scores given as they are.  The
// `extra` entries after them are gates of always-on parts: weights [top + extra] gets 1 for every chosen expert
// and the sigmoids of those entries.  `s` holds the logits on entry and is overwritten.
__device__ __forceinline__ void select_sigmoid_by_warp(float* s, int lane, int E, int extra, int top, int* ids,
                                                       float* scores, float* weights) {
  for (int e = lane; e < E + extra; e += 32) s[e] = 1.0f / (1.0f + expf(-s[e]));
  __syncwarp();
  for (int c = 0; c < top; ++c) {
    float val = -1.f;
    int idx = 0x7fffffff;
    for (int e = lane; e < E; e += 32)
      if (s[e] > val) { val = s[e]; idx = e; }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, val, o);
      const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
      if (ov > val || (ov == val && oi < idx)) { val = ov; idx = oi; }
    }
    if (lane == 0) {
      ids[c] = idx;
      scores[c] = val;
      weights[c] = 1.0f;
      s[idx] = -2.f;                          // taken
    }
    __syncwarp();
  }
  for (int e = lane; e < extra; e += 32) weights[top + e] = s[E + e];
}

// The choice of a sigmoid router limited to groups, by one warp, from float32 logits in shared memory: scores
// s = sigmoid(logit); choice scores c = s + correction (a learned offset per expert, or none); the E experts form
// n_groups equal groups of neighbours and a group scores as the sum of its two largest choice scores (of its one,
// if it has one member); only members of the `keep` best groups may be chosen (the others count as minus infinity:
// choice scores may be negative); the `top` largest choice scores of those are chosen (the lower index among equals).
// gates: the chosen experts' s, divided by their sum (+ 1e-20) if `normalize`, times out_scale.  `s` holds the logits
// on entry and the scores afterwards; `c` is scratch for E floats in shared memory.
__device__ __forceinline__ void select_sigmoid_grouped_by_warp(float* s, float* c, const float* __restrict__ correction,
                                                               int lane, int E, int top, int n_groups, int keep,
                                                               int normalize, float out_scale, int* ids, float* gates) {
  for (int e = lane; e < E; e += 32) {
    const float v = 1.0f / (1.0f + expf(-s[e]));
    s[e] = v;
    c[e] = correction ? v + correction[e] : v;
  }
  __syncwarp();
  auto best_of_warp = [&](float& val, int& idx) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, val, o);
      const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
      if (ov > val || (ov == val && oi < idx)) { val = ov; idx = oi; }
    }
  };
  const int per = E / n_groups;
  if (keep < n_groups) {
    float gs[2];                                  // the scores of groups lane and lane + 32
#pragma unroll
    for (int k = 0; k < 2; ++k) {
      const int g = lane + 32 * k;
      gs[k] = -INFINITY;
      if (g < n_groups) {
        float a = -INFINITY, b = -INFINITY;       // the two largest of the group
        for (int e = g * per; e < (g + 1) * per; ++e) {
          const float v = c[e];
          if (v > a) { b = a; a = v; } else if (v > b) { b = v; }
        }
        gs[k] = per > 1 ? a + b : a;
      }
    }
    unsigned long long kept = 0ull;
    for (int r = 0; r < keep; ++r) {
      float val = gs[0];
      int idx = lane < n_groups ? lane : 0x7fffffff;
      if (lane + 32 < n_groups && gs[1] > val) { val = gs[1]; idx = lane + 32; }
      best_of_warp(val, idx);
      kept |= 1ull << idx;
      if ((idx & 31) == lane) gs[idx >> 5] = -INFINITY;
    }
    __syncwarp();
    for (int e = lane; e < E; e += 32)
      if (!((kept >> (e / per)) & 1ull)) c[e] = -INFINITY;
    __syncwarp();
  }
  float my_val = 0.f, sum = 0.f;
  int my_sel = 0;
  for (int r = 0; r < top; ++r) {
    float val = -INFINITY;
    int idx = 0x7fffffff;
    for (int e = lane; e < E; e += 32)
      if (c[e] > val) { val = c[e]; idx = e; }
    best_of_warp(val, idx);
    const float sv = idx < E ? s[idx] : 0.f;
    if (lane == r) { my_val = sv; my_sel = idx < E ? idx : 0; }
    sum += sv;
    __syncwarp();
    if (lane == 0 && idx < E) c[idx] = -INFINITY;      // taken
    __syncwarp();
  }
  if (lane < top) {
    ids[lane] = my_sel;
    gates[lane] = (normalize ? my_val / (sum + 1e-20f) : my_val) * out_scale;
  }
}

}  // namespace flint
