// Router: logits = X W^T (float32 accumulate), sigmoid, + per-expert bias for selection,
// top-k with ties to the lower expert id, weights = raw score / max(sum, 1e-12) * scaling.
//
// Replaces native/cuda/kernels/router.cu:7-180 (one serial thread per row, or one CTA per
// (expert,row) dot product plus a global spin lock per row) with a tiled logits kernel and
// a one-warp-per-row selection kernel; there are no locks and no atomics, so the result is
// bit-reproducible.  Semantics follow python/reference/glmrt_reference/
// glm_moe_dsa_layer_ref.py:62-83 and, for non-finite scores, router.cu:112-116.
#include <math_constants.h>

#include <mutex>

#include "common.cuh"
#include "internal.h"
#include "plan_body.cuh"

GLMRT_CHAIN_TRACE_TU(router)

namespace glmrt {
namespace {

constexpr int kTM = 64;    // rows per CTA
constexpr int kTN = 4;     // experts per CTA
constexpr int kKC = 128;   // K chunk staged in shared memory
constexpr size_t kMaxRouterTopK = 64;  // native/cuda/kernels/common.h:18

template <typename T>
__device__ __forceinline__ float load_as_f32(const T* p, size_t i);
template <>
__device__ __forceinline__ float load_as_f32<float>(const float* p, size_t i) { return p[i]; }
template <>
__device__ __forceinline__ float load_as_f32<uint16_t>(const uint16_t* p, size_t i) {
  return bf16_bits_to_f32(p[i]);
}

// logits[row, expert] = sum_k x[row, k] * w[expert, k], float32 FMA in ascending k.
template <typename XT, typename WT>
__global__ void __launch_bounds__(kTM * kTN)
router_logits_kernel(const XT* __restrict__ x, const WT* __restrict__ w, float* __restrict__ logits,
                     int rows, int hidden, int experts) {
  __shared__ float xs[kKC][kTM + 1];
  __shared__ float ws[kTN][kKC];
  const int tm = threadIdx.x % kTM;
  const int tn = threadIdx.x / kTM;
  const int row0 = blockIdx.x * kTM;
  const int exp0 = blockIdx.y * kTN;
  float acc = 0.0f;
  for (int k0 = 0; k0 < hidden; k0 += kKC) {
    const int kc = min(kKC, hidden - k0);
    // stage X: coalesced along k
    for (int i = threadIdx.x; i < kTM * kKC; i += kTM * kTN) {
      const int r = i / kKC, k = i % kKC;
      float v = 0.0f;
      if (row0 + r < rows && k < kc) v = load_as_f32<XT>(x, static_cast<size_t>(row0 + r) * hidden + k0 + k);
      xs[k][r] = v;
    }
    for (int i = threadIdx.x; i < kTN * kKC; i += kTM * kTN) {
      const int e = i / kKC, k = i % kKC;
      float v = 0.0f;
      if (exp0 + e < experts && k < kc) v = load_as_f32<WT>(w, static_cast<size_t>(exp0 + e) * hidden + k0 + k);
      ws[e][k] = v;
    }
    __syncthreads();
#pragma unroll 8
    for (int k = 0; k < kKC; ++k) acc = fmaf(xs[k][tm], ws[tn][k], acc);
    __syncthreads();
  }
  if (row0 + tm < rows && exp0 + tn < experts)
    logits[static_cast<size_t>(row0 + tm) * experts + exp0 + tn] = acc;
}

// Decode-sized batches: one CTA per pair of experts, each warp takes four rows per pass and its
// lanes split the reduction dimension, so the float32 router weight is streamed from HBM exactly
// once by 128 CTAs while the few activation rows are served by L2.  hidden % 128 == 0.
// The per-lane partial sums and the butterfly reduction have a fixed order: results are
// bit-reproducible.
template <typename WT>
__device__ __forceinline__ float4 load_w4(const WT* p);
template <>
__device__ __forceinline__ float4 load_w4<float>(const float* p) {
  return __ldg(reinterpret_cast<const float4*>(p));
}
template <>
__device__ __forceinline__ float4 load_w4<uint16_t>(const uint16_t* p) {
  const uint2 v = __ldg(reinterpret_cast<const uint2*>(p));
  return make_float4(__uint_as_float(v.x << 16), __uint_as_float(v.x & 0xffff0000u),
                     __uint_as_float(v.y << 16), __uint_as_float(v.y & 0xffff0000u));
}

constexpr int kSmallThreads = 512;   // 16 warps
constexpr int kSmallWarps = kSmallThreads / 32;
constexpr int kSmallRows = 4;        // rows per pass
constexpr int kSmallMaxRows = 128;
constexpr int kSmallMaxSteps = 4;     // 128-element steps per warp: hidden <= 8192
constexpr int kSmallExperts = 4;      // experts per CTA
constexpr int kSmallChunkRows = 64;   // rows per CTA (the batch is cut in two from eight rows on)

// One CTA computes kSmallExperts experts for one chunk of the rows.  The 128-element steps of the
// reduction are dealt round-robin to the 16 warps; each warp keeps its slice of the weight rows in
// registers and sweeps the chunk's rows, then the 16 partial sums of every logit are added in warp
// order.  The summation order depends on hidden only, never on the number of rows or on how they
// are cut into chunks, so a row routed alone gets the same logits as inside any batch.  What a CTA
// reads is bounded by the rate one SM takes data from L2, so four experts share each pass over
// the rows and the rows are shared out between two CTAs (half the bytes per CTA of a two-expert,
// all-rows CTA; with the rotated row order measured 0.045 -> 0.035 ms at 64 rows).
template <typename WT>
__global__ void __launch_bounds__(kSmallThreads)
router_logits_small_kernel(const uint16_t* __restrict__ x, const WT* __restrict__ w, float* __restrict__ logits,
                           int rows, int hidden, int experts, int chunk_rows) {
  GLMRT_CHAIN_SCOPE(kChainLogits);
  pdl_launch_dependents();
  __shared__ float partial[kSmallWarps][kSmallChunkRows][kSmallExperts];
  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
  const int e0 = blockIdx.x * kSmallExperts;
  const int row0 = blockIdx.y * chunk_rows;
  const int nrows = min(chunk_rows, rows - row0);
  if (nrows <= 0) return;
  const int steps = hidden / 128;
  // this warp's slice of the weight rows stays in registers for the whole sweep over the rows.  The
  // router weight is a constant of the layer, not a result of the kernel in front: it is loaded
  // before griddepcontrol.wait, under that kernel's tail
  float4 wr[kSmallExperts][kSmallMaxSteps];
#pragma unroll
  for (int e = 0; e < kSmallExperts; ++e) {
    const WT* we = w + static_cast<size_t>(min(e0 + e, experts - 1)) * hidden;
#pragma unroll
    for (int s = 0; s < kSmallMaxSteps; ++s) {
      const int j = warp + s * kSmallWarps;
      wr[e][s] = j < steps ? load_w4<WT>(we + j * 128 + lane * 4) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
  }
  pdl_wait();   // the activation rows may be the previous kernel's output
  GLMRT_CHAIN_READY();
  GLMRT_CHAIN_MARK(0);
  // CTAs walk the row groups in rotated order: all of them reading the same activation lines at the
  // same moment would queue on a few L2 slices (a row's result does not depend on the order)
  const int groups = (nrows + kSmallRows - 1) / kSmallRows;
  const int first = static_cast<int>((blockIdx.x * 7u) % static_cast<unsigned>(groups));
  for (int g = 0; g < groups; ++g) {
    const int r0 = ((first + g) % groups) * kSmallRows;
    float acc[kSmallExperts][kSmallRows];
    uint2 px[kSmallMaxSteps][kSmallRows];
#pragma unroll
    for (int s = 0; s < kSmallMaxSteps; ++s) {
      const int j = warp + s * kSmallWarps;
#pragma unroll
      for (int i = 0; i < kSmallRows; ++i)
        px[s][i] = j < steps ? *reinterpret_cast<const uint2*>(
                                   x + static_cast<size_t>(row0 + min(r0 + i, nrows - 1)) * hidden + j * 128 + lane * 4)
                             : make_uint2(0u, 0u);
    }
#pragma unroll
    for (int e = 0; e < kSmallExperts; ++e)
#pragma unroll
      for (int i = 0; i < kSmallRows; ++i) acc[e][i] = 0.0f;
#pragma unroll
    for (int s = 0; s < kSmallMaxSteps; ++s) {
#pragma unroll
      for (int i = 0; i < kSmallRows; ++i) {
        const uint2 p = px[s][i];
        const float x0 = __uint_as_float(p.x << 16), x1 = __uint_as_float(p.x & 0xffff0000u);
        const float x2 = __uint_as_float(p.y << 16), x3 = __uint_as_float(p.y & 0xffff0000u);
#pragma unroll
        for (int e = 0; e < kSmallExperts; ++e) {
          float a = acc[e][i];
          a = fmaf(x0, wr[e][s].x, a); a = fmaf(x1, wr[e][s].y, a);
          a = fmaf(x2, wr[e][s].z, a); a = fmaf(x3, wr[e][s].w, a);
          acc[e][i] = a;
        }
      }
    }
#pragma unroll
    for (int i = 0; i < kSmallRows; ++i) {
#pragma unroll
      for (int e = 0; e < kSmallExperts; ++e) {
        float a = acc[e][i];
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) a += __shfl_xor_sync(0xffffffffu, a, off);
        if (lane == 0 && r0 + i < nrows) partial[warp][r0 + i][e] = a;
      }
    }
  }
  __syncthreads();
  GLMRT_CHAIN_MARK(1);
  for (int t = threadIdx.x; t < nrows * kSmallExperts; t += kSmallThreads) {
    const int r = t / kSmallExperts, e = t % kSmallExperts;
    float sum = 0.0f;
#pragma unroll
    for (int wv = 0; wv < kSmallWarps; ++wv) sum += partial[wv][r][e];
    if (e0 + e < experts) logits[static_cast<size_t>(row0 + r) * experts + e0 + e] = sum;
  }
}

// One warp per row.  Shared memory: per warp 2 * `experts` floats (used above 256 experts; up to
// 256 a lane keeps its eight experts in registers).
constexpr int kSelectPerLane = 8;
// Order-preserving integer key of a selection score (-0 and +0 get the same key, as they compare
// equal); -inf, the mark of an entry that must never be picked, gets the lowest key of all.
constexpr uint32_t kSelectNoKey = 0x007fffffu;   // key of -inf
__device__ __forceinline__ uint32_t select_key(float v) {
  const uint32_t bits = __float_as_uint(v + 0.0f);
  return (bits & 0x80000000u) ? ~bits : (bits | 0x80000000u);
}
__global__ void router_select_kernel(const float* __restrict__ logits, const float* __restrict__ bias,
                                     uint32_t* __restrict__ topk_indices, float* __restrict__ topk_scores,
                                     float* __restrict__ topk_weights, int rows, int experts, int top_k,
                                     float scaling, int splits, RouterCountTail tail) {
  GLMRT_CHAIN_SCOPE(kChainSelect);
  pdl_launch_dependents();
  pdl_wait();
  GLMRT_CHAIN_READY();
  extern __shared__ float smem[];
  const int warps = blockDim.x / 32;
  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
  const int row = blockIdx.x * warps + warp;
  if (row < rows) {
  float* sel = smem + static_cast<size_t>(warp) * 2 * experts;
  float* raw = sel + experts;
  const bool in_regs = experts <= 32 * kSelectPerLane;   // GLM-5.2's 256 experts: eight per lane
  // register path: the lane's experts j * 32 + lane as (order-preserving key of the selection score,
  // expert id, raw score)
  uint32_t vkey[kSelectPerLane], vid[kSelectPerLane];
  float vraw[kSelectPerLane];
  for (int base = 0; base < experts; base += 32 * kSelectPerLane) {
    // All loads of a pass are issued before any is used: one memory round trip per 256 experts
    // instead of one per expert.  A logit may arrive as `splits` partial sums (tensor-core router
    // below one wave of tiles): added in order.
    float lg[kSelectPerLane], bs[kSelectPerLane];
#pragma unroll
    for (int j = 0; j < kSelectPerLane; ++j) {
      const int e = base + j * 32 + lane;
      lg[j] = e < experts ? logits[static_cast<size_t>(row) * experts + e] : 0.0f;
      bs[j] = e < experts ? bias[e] : 0.0f;
    }
    const size_t stride = static_cast<size_t>(rows) * experts;
    for (int sp = 1; sp < splits; ++sp) {
      float v[kSelectPerLane];
#pragma unroll
      for (int j = 0; j < kSelectPerLane; ++j) {
        const int e = base + j * 32 + lane;
        v[j] = e < experts ? logits[sp * stride + static_cast<size_t>(row) * experts + e] : 0.0f;
      }
#pragma unroll
      for (int j = 0; j < kSelectPerLane; ++j) lg[j] = __fadd_rn(lg[j], v[j]);
    }
#pragma unroll
    for (int j = 0; j < kSelectPerLane; ++j) {
      const int e = base + j * 32 + lane;
      const float sg = sigmoid_f32(lg[j]);
      const bool fin = isfinite(sg);
      const float score = fin ? sg : 0.0f;
      const float corrected = score + bs[j];
      const float pick = (fin && isfinite(corrected) && e < experts) ? corrected : -CUDART_INF_F;
      if (in_regs) {
        vraw[j] = score;
        vid[j] = static_cast<uint32_t>(e);
        vkey[j] = select_key(pick);
      } else if (e < experts) {
        raw[e] = score;
        sel[e] = pick;
      }
    }
  }
  __syncwarp();
  GLMRT_CHAIN_MARK(0);
  if (in_regs) {
    // The lane's eight candidates are sorted once (best first; equal scores: lower expert first), so
    // that every rank below looks at the lane's head only.  19 compare-exchanges, four at a time.
    auto order = [&](int i, int j) {
      const bool swap = vkey[j] > vkey[i] || (vkey[j] == vkey[i] && vid[j] < vid[i]);
      const uint32_t ki = vkey[i], ii = vid[i];
      const float ri = vraw[i];
      vkey[i] = swap ? vkey[j] : ki; vid[i] = swap ? vid[j] : ii; vraw[i] = swap ? vraw[j] : ri;
      vkey[j] = swap ? ki : vkey[j]; vid[j] = swap ? ii : vid[j]; vraw[j] = swap ? ri : vraw[j];
    };
    static_assert(kSelectPerLane == 8, "the sorting network below is the 8-input one");
    order(0, 1); order(2, 3); order(4, 5); order(6, 7);
    order(0, 2); order(1, 3); order(4, 6); order(5, 7);
    order(1, 2); order(5, 6); order(0, 4); order(3, 7);
    order(1, 5); order(2, 6);
    order(1, 4); order(3, 6);
    order(2, 4); order(3, 5);
    order(3, 4);
  }
  float sum = 0.0f;
  float my_score = 0.0f;   // lane j keeps the score of rank j (top_k <= 64: two per lane)
  float my_score2 = 0.0f;
  uint32_t my_idx = 0, my_idx2 = 0;
  for (int rank = 0; rank < top_k; ++rank) {
    float score = 0.0f;
    uint32_t idx = 0;
    if (in_regs) {
      // two warp reductions over the lanes' heads: the largest key, and the lowest expert among the
      // lanes that hold it; the winning lane moves on to its next candidate
      const uint32_t top = __reduce_max_sync(0xffffffffu, vkey[0]);
      const uint32_t cand = (vkey[0] == top && top != kSelectNoKey) ? vid[0] : 0x7fffffffu;
      const uint32_t win = __reduce_min_sync(0xffffffffu, cand);
      if (win != 0x7fffffffu) {   // a finite candidate exists
        score = __shfl_sync(0xffffffffu, vraw[0], static_cast<int>(win & 31u));
        idx = win;
        if (lane == static_cast<int>(win & 31u)) {
#pragma unroll
          for (int j = 0; j + 1 < kSelectPerLane; ++j) { vkey[j] = vkey[j + 1]; vid[j] = vid[j + 1]; vraw[j] = vraw[j + 1]; }
          vkey[kSelectPerLane - 1] = kSelectNoKey;
        }
      }
    } else {
      float best = -CUDART_INF_F;
      int best_e = 0x7fffffff;
      for (int e = lane; e < experts; e += 32) {
        const float v = sel[e];
        if (v > best) { best = v; best_e = e; }   // ascending e: first maximum wins inside a lane
      }
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) {
        const float ob = __shfl_xor_sync(0xffffffffu, best, off);
        const int oe = __shfl_xor_sync(0xffffffffu, best_e, off);
        if (ob > best || (ob == best && oe < best_e)) { best = ob; best_e = oe; }
      }
      if (best_e != 0x7fffffff) {  // a finite candidate exists
        score = raw[best_e];
        idx = static_cast<uint32_t>(best_e);
        if (lane == 0) sel[best_e] = -CUDART_INF_F;  // -inf entries are never picked (best starts at -inf)
      }
      __syncwarp();
    }
    sum += score;  // sequential float32 sum in rank order (router.cu:52-56)
    if (rank == lane) { my_score = score; my_idx = idx; }
    if (rank == lane + 32) { my_score2 = score; my_idx2 = idx; }
  }
  sum = fmaxf(sum, 1.0e-12f);
  const size_t out = static_cast<size_t>(row) * top_k;
  if (lane < top_k) {
    topk_indices[out + lane] = my_idx;
    if (topk_scores != nullptr) topk_scores[out + lane] = my_score;
    topk_weights[out + lane] = my_score / sum * scaling;
  }
  if (lane + 32 < top_k) {
    topk_indices[out + lane + 32] = my_idx2;
    if (topk_scores != nullptr) topk_scores[out + lane + 32] = my_score2;
    topk_weights[out + lane + 32] = my_score2 / sum * scaling;
  }
  }  // row < rows
  GLMRT_CHAIN_MARK(1);
  if (tail.ticket == nullptr) return;
  // The last CTA to finish does what would otherwise be a launch of its own: on the
  // expert-parallel path it counts this rank's routes per expert and publishes the histogram to
  // every rank (the first step of the exchange); on one GPU it builds the route plan.
  if (gridDim.x > 1) {
    __shared__ int s_is_last;
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) s_is_last = atomicAdd(tail.ticket, 1) == static_cast<int>(gridDim.x) - 1;
    __syncthreads();
    if (!s_is_last) return;
    __threadfence();
  } else {
    __syncthreads();   // a grid of one CTA: its own rows are all there are
  }
  GLMRT_CHAIN_MARK(2);
  if (tail.do_plan) {
    if (threadIdx.x == 0) *tail.ticket = 0;
    route_plan_body(tail.plan, blockDim.x);
    return;
  }
  int* hist = reinterpret_cast<int*>(smem);   // 2 * experts floats per warp are free again
  for (int e = threadIdx.x; e < experts; e += blockDim.x) hist[e] = 0;
  __syncthreads();
  const int routes = rows * top_k;
  const volatile uint32_t* all_idx = topk_indices;   // written by other CTAs of this grid
  for (int r = threadIdx.x; r < routes; r += blockDim.x) {
    const uint32_t e = all_idx[r];
    // the count so far is the route's position among this rank's routes of that expert: the push
    // kernel needs no counter of its own
    const int pos = e < static_cast<uint32_t>(experts) ? atomicAdd(&hist[e], 1) : -1;
    if (tail.route_pos != nullptr) tail.route_pos[r] = pos;
  }
  __syncthreads();
  for (int e = threadIdx.x; e < experts; e += blockDim.x) {
    const int c = hist[e];
    for (int p = 0; p < tail.world; ++p) tail.peer_counts[p][e] = c;
  }
  if (threadIdx.x == 0) {
    *tail.error_word = 0u;   // a new step begins: clear the layer's error word
    *tail.ticket = 0;
  }
  __syncthreads();   // the release below is cumulative over what the barrier ordered before it
  if (threadIdx.x < static_cast<unsigned>(tail.world)) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(tail.peer_flags[threadIdx.x]), "r"(tail.epoch) : "memory");
  }
}

glmrt_status_t validate(const void* hidden, const void* weight, const float* bias, const uint32_t* idx,
                        const float* weights, size_t rows, size_t hidden_dim, size_t experts, size_t top_k) {
  if (hidden == nullptr || weight == nullptr || bias == nullptr || idx == nullptr || weights == nullptr)
    return fail(GLMRT_STATUS_INVALID_ARGUMENT, "router: null pointer argument");
  if (rows == 0 || hidden_dim == 0 || experts == 0 || top_k == 0 || top_k > experts || top_k > kMaxRouterTopK)
    return fail(GLMRT_STATUS_INVALID_ARGUMENT, "router: rows, hidden_dim, experts must be > 0 and 0 < top_k <= min(experts, 64)");
  size_t ignored = 0;
  if (!checked_mul(rows, hidden_dim, &ignored) || !checked_mul(experts, hidden_dim, &ignored) ||
      !checked_mul(rows, experts, &ignored) || rows > static_cast<size_t>(std::numeric_limits<int>::max()) ||
      experts > 1024 || hidden_dim > static_cast<size_t>(std::numeric_limits<int>::max()))
    return fail(GLMRT_STATUS_INVALID_ARGUMENT, "router: dimensions out of range");
  return GLMRT_STATUS_OK;
}

}  // namespace

glmrt_status_t launch_router(const void* hidden, bool hidden_bf16, const void* weight, bool weight_bf16,
                             const float* bias, float* logits, uint32_t* idx, float* scores, float* weights,
                             size_t rows, size_t hidden_dim, size_t experts, size_t top_k, float scaling,
                             cudaStream_t stream, const RouterCountTail* tail) {
  const dim3 grid(static_cast<unsigned>((rows + kTM - 1) / kTM), static_cast<unsigned>((experts + kTN - 1) / kTN));
  const int r = static_cast<int>(rows), h = static_cast<int>(hidden_dim), e = static_cast<int>(experts);
  const bool small = hidden_bf16 && rows <= kSmallMaxRows && hidden_dim <= 128 * kSmallWarps * kSmallMaxSteps && hidden_dim % 128 == 0 &&
                     reinterpret_cast<uintptr_t>(hidden) % 8 == 0 && reinterpret_cast<uintptr_t>(weight) % 16 == 0;
  if (small) {
    // from eight rows on the rows are cut into two chunks (chunk sizes are multiples of the 4-row
    // pass): 128 CTAs instead of 64, each with half the passes; a row's logits do not depend on the cut
    const int chunk_rows = r < 8 ? r : std::min(kSmallChunkRows, ((r + 1) / 2 + kSmallRows - 1) / kSmallRows * kSmallRows);
    const dim3 ctas(static_cast<unsigned>((experts + kSmallExperts - 1) / kSmallExperts),
                    static_cast<unsigned>((r + chunk_rows - 1) / chunk_rows));
    if (weight_bf16)
      launch_pdl(router_logits_small_kernel<uint16_t>, ctas, dim3(kSmallThreads), 0, stream,
                 static_cast<const uint16_t*>(hidden), static_cast<const uint16_t*>(weight), logits, r, h, e, chunk_rows);
    else
      launch_pdl(router_logits_small_kernel<float>, ctas, dim3(kSmallThreads), 0, stream,
                 static_cast<const uint16_t*>(hidden), static_cast<const float*>(weight), logits, r, h, e, chunk_rows);
  } else if (hidden_bf16 && weight_bf16)
    router_logits_kernel<uint16_t, uint16_t><<<grid, kTM * kTN, 0, stream>>>(
        static_cast<const uint16_t*>(hidden), static_cast<const uint16_t*>(weight), logits, r, h, e);
  else if (hidden_bf16)
    router_logits_kernel<uint16_t, float><<<grid, kTM * kTN, 0, stream>>>(
        static_cast<const uint16_t*>(hidden), static_cast<const float*>(weight), logits, r, h, e);
  else if (!weight_bf16)
    router_logits_kernel<float, float><<<grid, kTM * kTN, 0, stream>>>(
        static_cast<const float*>(hidden), static_cast<const float*>(weight), logits, r, h, e);
  else
    return fail(GLMRT_STATUS_INVALID_ARGUMENT, "router: float32 hidden with bf16 weights is not supported");
  GLMRT_LAUNCH_CHECK("router_logits_kernel");
  return launch_router_select(logits, bias, idx, scores, weights, rows, experts, top_k, scaling, stream, 1, tail);
}

glmrt_status_t launch_router_select(const float* logits, const float* bias, uint32_t* idx, float* scores,
                                    float* weights, size_t rows, size_t experts, size_t top_k, float scaling,
                                    cudaStream_t stream, int splits, const RouterCountTail* tail) {
  const int warps = 4;
  RouterCountTail t{};
  if (tail != nullptr) t = *tail;
  const size_t smem = static_cast<size_t>(warps) * 2 * experts * sizeof(float);
  launch_pdl(router_select_kernel, dim3(static_cast<unsigned>((rows + warps - 1) / warps)), dim3(warps * 32), smem, stream,
             logits, bias, idx, scores, weights, static_cast<int>(rows), static_cast<int>(experts),
             static_cast<int>(top_k), scaling, splits, t);
  GLMRT_LAUNCH_CHECK("router_select_kernel");
  return GLMRT_STATUS_OK;
}

namespace {
// Entry points without a scratch argument take the logits buffer from the stream-ordered pool.
glmrt_status_t router_with_pool(const void* hidden, bool hidden_bf16, const void* weight, bool weight_bf16,
                                const float* bias, uint32_t* idx, float* scores, float* weights, size_t rows,
                                size_t hidden_dim, size_t experts, size_t top_k, cudaStream_t stream) {
  GLMRT_RETURN_IF_ERROR(validate(hidden, weight, bias, idx, weights, rows, hidden_dim, experts, top_k));
  if (scores == nullptr) return fail(GLMRT_STATUS_INVALID_ARGUMENT, "router: null pointer argument");
  GLMRT_RETURN_IF_ERROR(require_cuda());
  float* logits = nullptr;
  cudaError_t err = cudaMallocAsync(reinterpret_cast<void**>(&logits), rows * experts * sizeof(float), stream);
  if (err != cudaSuccess) return fail_cuda(GLMRT_STATUS_ALLOCATION_FAILED, "cudaMallocAsync", err);
  glmrt_status_t st = launch_router(hidden, hidden_bf16, weight, weight_bf16, bias, logits, idx, scores, weights,
                                    rows, hidden_dim, experts, top_k, 2.5f, stream);
  cudaFreeAsync(logits, stream);
  return st == GLMRT_STATUS_OK ? ok() : st;
}
}  // namespace
}  // namespace glmrt

using namespace glmrt;

extern "C" glmrt_status_t glmrt_cuda_router_topk_f32_async(
    const float* hidden, const float* router_weight, const float* correction_bias, uint32_t* topk_indices,
    float* topk_scores, float* topk_weights, size_t rows, size_t hidden_dim, size_t experts, size_t top_k,
    void* cuda_stream) {
  return router_with_pool(hidden, false, router_weight, false, correction_bias, topk_indices, topk_scores,
                          topk_weights, rows, hidden_dim, experts, top_k, static_cast<cudaStream_t>(cuda_stream));
}
extern "C" glmrt_status_t glmrt_cuda_router_topk_f32(const float* hidden, const float* router_weight,
                                                     const float* correction_bias, uint32_t* topk_indices,
                                                     float* topk_scores, float* topk_weights, size_t rows,
                                                     size_t hidden_dim, size_t experts, size_t top_k) {
  GLMRT_RETURN_IF_ERROR(glmrt_cuda_router_topk_f32_async(hidden, router_weight, correction_bias, topk_indices,
                                                         topk_scores, topk_weights, rows, hidden_dim, experts,
                                                         top_k, nullptr));
  return status_from_cuda(cudaStreamSynchronize(nullptr), "cudaStreamSynchronize");
}
extern "C" glmrt_status_t glmrt_cuda_router_topk_bf16_async(
    const uint16_t* hidden, const uint16_t* router_weight, const float* correction_bias, uint32_t* topk_indices,
    float* topk_scores, float* topk_weights, size_t rows, size_t hidden_dim, size_t experts, size_t top_k,
    void* cuda_stream) {
  return router_with_pool(hidden, true, router_weight, true, correction_bias, topk_indices, topk_scores,
                          topk_weights, rows, hidden_dim, experts, top_k, static_cast<cudaStream_t>(cuda_stream));
}
extern "C" glmrt_status_t glmrt_cuda_router_topk_bf16(const uint16_t* hidden, const uint16_t* router_weight,
                                                      const float* correction_bias, uint32_t* topk_indices,
                                                      float* topk_scores, float* topk_weights, size_t rows,
                                                      size_t hidden_dim, size_t experts, size_t top_k) {
  GLMRT_RETURN_IF_ERROR(glmrt_cuda_router_topk_bf16_async(hidden, router_weight, correction_bias, topk_indices,
                                                          topk_scores, topk_weights, rows, hidden_dim, experts,
                                                          top_k, nullptr));
  return status_from_cuda(cudaStreamSynchronize(nullptr), "cudaStreamSynchronize");
}
// The reference's variant with caller-owned scratch (no allocation, so it can be captured in a CUDA
// graph; native/cuda/kernels/router.cu:582-644 sorts every row with a segmented radix sort).  Here
// the same selection kernel as everywhere runs on logits kept in `corrected_scores`; the other
// scratch arrays are validated like the reference does and left untouched.
extern "C" glmrt_status_t glmrt_cuda_router_topk_bf16_cub_async(
    const uint16_t* hidden, const uint16_t* router_weight, const float* correction_bias, float* corrected_scores,
    float* sorted_corrected_scores, uint32_t* unsorted_indices, uint32_t* sorted_indices, int* segment_offsets,
    uint32_t* topk_indices, float* topk_scores, float* topk_weights, void* cub_temp_storage,
    size_t cub_temp_storage_bytes, size_t rows, size_t hidden_dim, size_t experts, size_t top_k, void* cuda_stream) {
  GLMRT_RETURN_IF_ERROR(validate(hidden, router_weight, correction_bias, topk_indices, topk_weights, rows, hidden_dim,
                                 experts, top_k));
  if (topk_scores == nullptr || corrected_scores == nullptr || sorted_corrected_scores == nullptr ||
      unsorted_indices == nullptr || sorted_indices == nullptr || segment_offsets == nullptr ||
      cub_temp_storage == nullptr || cub_temp_storage_bytes == 0)
    return fail(GLMRT_STATUS_INVALID_ARGUMENT, "router (caller scratch): null scratch pointer or empty temporary storage");
  if (rows * experts > static_cast<size_t>(std::numeric_limits<int>::max()))
    return fail(GLMRT_STATUS_INVALID_ARGUMENT, "router (caller scratch): rows * experts out of range");
  GLMRT_RETURN_IF_ERROR(require_cuda());
  GLMRT_RETURN_IF_ERROR(launch_router(hidden, true, router_weight, true, correction_bias, corrected_scores, topk_indices,
                                      topk_scores, topk_weights, rows, hidden_dim, experts, top_k, 2.5f,
                                      static_cast<cudaStream_t>(cuda_stream)));
  return ok();
}
extern "C" glmrt_status_t glmrt_cuda_router_topk_bf16_cub(
    const uint16_t* hidden, const uint16_t* router_weight, const float* correction_bias, float* corrected_scores,
    float* sorted_corrected_scores, uint32_t* unsorted_indices, uint32_t* sorted_indices, int* segment_offsets,
    uint32_t* topk_indices, float* topk_scores, float* topk_weights, void* cub_temp_storage,
    size_t cub_temp_storage_bytes, size_t rows, size_t hidden_dim, size_t experts, size_t top_k) {
  GLMRT_RETURN_IF_ERROR(glmrt_cuda_router_topk_bf16_cub_async(
      hidden, router_weight, correction_bias, corrected_scores, sorted_corrected_scores, unsorted_indices,
      sorted_indices, segment_offsets, topk_indices, topk_scores, topk_weights, cub_temp_storage,
      cub_temp_storage_bytes, rows, hidden_dim, experts, top_k, nullptr));
  return status_from_cuda(cudaStreamSynchronize(nullptr), "cudaStreamSynchronize");
}
extern "C" glmrt_status_t glmrt_b200_router_topk_bf16_f32w_async(
    const uint16_t* hidden, const float* router_weight, const float* correction_bias, float* logits_scratch,
    uint32_t* topk_indices, float* topk_scores, float* topk_weights, size_t rows, size_t hidden_dim,
    size_t experts, size_t top_k, void* cuda_stream) {
  GLMRT_RETURN_IF_ERROR(validate(hidden, router_weight, correction_bias, topk_indices, topk_weights, rows,
                                 hidden_dim, experts, top_k));
  if (logits_scratch == nullptr) return fail(GLMRT_STATUS_INVALID_ARGUMENT, "router: logits scratch is null");
  GLMRT_RETURN_IF_ERROR(require_cuda());
  GLMRT_RETURN_IF_ERROR(launch_router(hidden, true, router_weight, false, correction_bias, logits_scratch,
                                      topk_indices, topk_scores, topk_weights, rows, hidden_dim, experts, top_k,
                                      2.5f, static_cast<cudaStream_t>(cuda_stream)));
  return ok();
}

// ---- allocation-free variant -------------------------------------------------------------
// Logits scratch that lives in the library image instead of in allocated memory.  Every GPU that
// loads the library holds these 1 MiB until the process exits.
namespace {
constexpr size_t kStaticLogitsFloats = 262144;  // rows * experts may not exceed this
static __device__ __align__(256) float g_static_logits[kStaticLogitsFloats];

constexpr int kMaxDevices = 64;
std::mutex g_static_mu;
float* g_static_ptr[kMaxDevices] = {};

// Device address of g_static_logits on the current device.  In host code the symbol's name is
// only a handle; the address a kernel can use has to be asked for, once per device, while that
// device is current.
glmrt_status_t static_logits_ptr(float** out) {
  int dev = 0;
  cudaError_t err = cudaGetDevice(&dev);
  if (err != cudaSuccess) return fail_cuda(GLMRT_STATUS_INTERNAL_ERROR, "cudaGetDevice", err);
  if (dev < 0 || dev >= kMaxDevices) return fail(GLMRT_STATUS_INVALID_ARGUMENT, "router (static scratch): device index out of range");
  std::lock_guard<std::mutex> lock(g_static_mu);
  if (g_static_ptr[dev] == nullptr) {
    float* p = nullptr;
    err = cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_static_logits);
    if (err != cudaSuccess || p == nullptr)
      return fail_cuda(GLMRT_STATUS_INTERNAL_ERROR, "cudaGetSymbolAddress(static logits scratch)", err);
    g_static_ptr[dev] = p;
  }
  *out = g_static_ptr[dev];
  return GLMRT_STATUS_OK;
}
}  // namespace

extern "C" glmrt_status_t glmrt_b200_router_topk_bf16_f32w_static_async(
    const uint16_t* hidden, const float* router_weight, const float* correction_bias, uint32_t* topk_indices,
    float* topk_scores, float* topk_weights, size_t rows, size_t hidden_dim, size_t experts, size_t top_k,
    void* cuda_stream) {
  GLMRT_RETURN_IF_ERROR(validate(hidden, router_weight, correction_bias, topk_indices, topk_weights, rows,
                                 hidden_dim, experts, top_k));
  if (rows * experts > kStaticLogitsFloats)
    return fail(GLMRT_STATUS_BUFFER_TOO_SMALL,
                "router (static scratch): rows * experts exceeds the built-in scratch of 262144 floats; use "
                "glmrt_b200_router_topk_bf16_f32w_async with caller-provided scratch");
  GLMRT_RETURN_IF_ERROR(require_cuda());
  float* logits = nullptr;
  GLMRT_RETURN_IF_ERROR(static_logits_ptr(&logits));
  // Every logit the selection kernel reads is written by the logits kernel of the same call, so
  // nothing left behind by an earlier call has to be cleared.
  GLMRT_RETURN_IF_ERROR(launch_router(hidden, true, router_weight, false, correction_bias, logits, topk_indices,
                                      topk_scores, topk_weights, rows, hidden_dim, experts, top_k, 2.5f,
                                      static_cast<cudaStream_t>(cuda_stream)));
  return ok();
}
