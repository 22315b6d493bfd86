// Detection post-processing and evaluation on the device: pairwise box IoU, greedy class-aware NMS, confusion matrices,
// binary mask counts, segmentation metrics and dataset-level detection metrics (greedy matching, precision / recall curves,
// 101-point interpolated AP, mAP).  Contract: Source/Public/Oa/Vision/FnDetection.h and the shaders under
// Source/Private/Oa/Vision/Shader/Compute/Postprocess of the reference, which run NMS and the metric curves on a single
// thread; here every selection (best candidate, best target) is a block-wide arg-max with the same tie rule (higher value,
// then lower index), so the results are identical and the scan over candidates is parallel.
#include "common.cuh"
#include "api.h"

namespace oa {

__device__ __forceinline__ float box_iou_cxcywh(const float* __restrict__ a, const float* __restrict__ b) {
  const float aw = fmaxf(a[2], 0.f), ah = fmaxf(a[3], 0.f), bw = fmaxf(b[2], 0.f), bh = fmaxf(b[3], 0.f);
  const float ix = fmaxf(fminf(a[0] + aw * 0.5f, b[0] + bw * 0.5f) - fmaxf(a[0] - aw * 0.5f, b[0] - bw * 0.5f), 0.f);
  const float iy = fmaxf(fminf(a[1] + ah * 0.5f, b[1] + bh * 0.5f) - fmaxf(a[1] - ah * 0.5f, b[1] - bh * 0.5f), 0.f);
  const float inter = ix * iy, uni = aw * ah + bw * bh - inter;
  return uni > 0.f ? inter / uni : 0.f;
}

__global__ void box_iou_kernel(const float* __restrict__ a, const float* __restrict__ b, float* __restrict__ out, int n, int m) {
  const long long total = (long long)n * m;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int r = (int)(i / m), c = (int)(i % m);
    out[i] = box_iou_cxcywh(a + 4 * r, b + 4 * c);
  }
}

// Block-wide arg-max of (value, lower index wins ties); every thread gets the winner.  idx = -1 means "no candidate".
struct Best { float v; int idx; };
__device__ __forceinline__ Best better(Best a, Best b) {
  if (b.idx < 0) return a;
  if (a.idx < 0) return b;
  if (b.v > a.v || (b.v == a.v && b.idx < a.idx)) return b;
  return a;
}
__device__ Best block_argmax(Best mine, Best* scratch) {
  for (int o = 16; o > 0; o >>= 1) {
    Best other;
    other.v = __shfl_xor_sync(0xffffffffu, mine.v, o);
    other.idx = __shfl_xor_sync(0xffffffffu, mine.idx, o);
    mine = better(mine, other);
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
  __syncthreads();
  if (lane == 0) scratch[warp] = mine;
  __syncthreads();
  Best r = scratch[0];
  for (int w = 1; w < warps; ++w) r = better(r, scratch[w]);
  return r;
}

// One CTA.  alive[] (global scratch, n bytes) marks candidates still selectable.  Each round: pick the best alive candidate,
// record it, then drop every alive candidate of the same class (or any class) whose IoU with it reaches the threshold.
__global__ void __launch_bounds__(1024) nms_kernel(const float* __restrict__ boxes, const float* __restrict__ scores,
                                                   const int* __restrict__ classes, int n, float iou_thr, float score_thr, int max_det,
                                                   int agnostic, int* __restrict__ indices, unsigned* __restrict__ count,
                                                   unsigned char* __restrict__ alive) {
  __shared__ Best scratch[32];
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const float s = scores[i];
    alive[i] = (s == s && s >= score_thr) ? 1 : 0;
    indices[i] = -1;
  }
  __syncthreads();
  int selected = 0;
  const int limit = max_det < n ? max_det : n;
  for (int round = 0; round < limit; ++round) {
    Best mine{0.f, -1};
    for (int i = threadIdx.x; i < n; i += blockDim.x)
      if (alive[i]) mine = better(mine, Best{scores[i], i});
    const Best win = block_argmax(mine, scratch);
    if (win.idx < 0) break;
    const int wc = classes[win.idx];
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
      if (!alive[i]) continue;
      if (i == win.idx || ((agnostic || classes[i] == wc) && box_iou_cxcywh(boxes + 4 * i, boxes + 4 * win.idx) >= iou_thr)) alive[i] = 0;
    }
    if (threadIdx.x == 0) indices[selected] = win.idx;
    ++selected;
    __syncthreads();
  }
  if (threadIdx.x == 0) *count = (unsigned)selected;
}

__global__ void confusion_kernel(const int* __restrict__ predicted, const int* __restrict__ target, long long n, int classes,
                                 unsigned* __restrict__ out) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const int p = predicted[i], t = target[i];
    if (p >= 0 && p < classes && t >= 0 && t < classes) atomicAdd(out + (long long)t * classes + p, 1u);
  }
}

// out[4] = true positive, false positive, false negative, true negative over uint8 masks (non-zero = set)
__global__ void binary_counts_kernel(const unsigned char* __restrict__ predicted, const unsigned char* __restrict__ target, long long n,
                                     unsigned* __restrict__ out) {
  unsigned c[4] = {0u, 0u, 0u, 0u};
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const bool p = predicted[i] != 0, t = target[i] != 0;
    c[p ? (t ? 0 : 1) : (t ? 2 : 3)]++;
  }
  for (int k = 0; k < 4; ++k) {
    unsigned v = c[k];
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    if ((threadIdx.x & 31) == 0 && v) atomicAdd(out + k, v);
  }
}

// One CTA: per-class precision / recall / F1 / IoU from a [C,C] confusion matrix (rows = target), mean IoU over classes
// with a non-empty union, pixel accuracy.
__global__ void segmentation_metrics_kernel(const unsigned* __restrict__ confusion, int classes, float* __restrict__ per_class,
                                            float* __restrict__ mean_iou, float* __restrict__ accuracy) {
  for (int c = threadIdx.x; c < classes; c += blockDim.x) {
    const unsigned tp = confusion[(long long)c * classes + c];
    unsigned tt = 0u, pt = 0u;
    for (int o = 0; o < classes; ++o) {
      tt += confusion[(long long)c * classes + o];
      pt += confusion[(long long)o * classes + c];
    }
    const unsigned fp = pt - tp, fn = tt - tp, uni = tp + fp + fn;
    const float precision = pt ? (float)tp / (float)pt : 0.f, recall = tt ? (float)tp / (float)tt : 0.f;
    const float f1 = precision + recall > 0.f ? 2.f * precision * recall / (precision + recall) : 0.f;
    const float iou = uni ? (float)tp / (float)uni : 0.f;
    per_class[c * 4 + 0] = precision; per_class[c * 4 + 1] = recall; per_class[c * 4 + 2] = f1; per_class[c * 4 + 3] = iou;
  }
  __syncthreads();
  if (threadIdx.x == 0) {                                   // sequential, in class order: the sums are reproducible
    float iou_sum = 0.f;
    unsigned valid = 0u, total = 0u, correct = 0u;
    for (int c = 0; c < classes; ++c) {
      const unsigned tp = confusion[(long long)c * classes + c];
      unsigned tt = 0u, pt = 0u;
      for (int o = 0; o < classes; ++o) {
        tt += confusion[(long long)c * classes + o];
        pt += confusion[(long long)o * classes + c];
      }
      if (tt + pt - tp) { iou_sum += per_class[c * 4 + 3]; ++valid; }
      total += tt;
      correct += tp;
    }
    *mean_iou = valid ? iou_sum / (float)valid : 0.f;
    *accuracy = total ? (float)correct / (float)total : 0.f;
  }
}

// One CTA per (threshold, class).  order[] lists predictions by descending score (ties: ascending index).  Greedy matching in
// that order against unmatched targets of the same class and image; curve[pair, rank] = (precision, recall).
__global__ void __launch_bounds__(256) detection_curves_kernel(
    const float* __restrict__ pboxes, const float* __restrict__ pscores, const int* __restrict__ pclasses, const int* __restrict__ pimages,
    const int* __restrict__ order, int P, const float* __restrict__ tboxes, const int* __restrict__ tclasses, const int* __restrict__ timages,
    int G, const float* __restrict__ thresholds, int classes, float score_thr, unsigned char* __restrict__ matched,
    float* __restrict__ curve, unsigned* __restrict__ counts, float* __restrict__ metrics) {
  __shared__ Best scratch[8];
  __shared__ unsigned target_count;
  const int pair = blockIdx.x, ti = pair / classes, cls = pair - ti * classes;
  const float thr = thresholds[ti];
  const bool thr_ok = thr == thr && thr >= 0.f && thr <= 1.f;
  unsigned char* used = matched + (long long)pair * G;
  float* cv = curve + (long long)pair * P * 2;
  if (threadIdx.x == 0) target_count = 0u;
  __syncthreads();
  unsigned local = 0u;
  for (int g = threadIdx.x; g < G; g += blockDim.x) {
    used[g] = 0;
    if (tclasses[g] == cls) ++local;
  }
  for (int r = threadIdx.x; r < P; r += blockDim.x) { cv[2 * r] = 0.f; cv[2 * r + 1] = 0.f; }
  if (local) atomicAdd(&target_count, local);
  __syncthreads();
  const unsigned targets = target_count;
  unsigned tp = 0u, fp = 0u, etp = 0u, efp = 0u;
  int rank = 0;
  for (int k = 0; k < P; ++k) {
    const int p = order[k];
    const float s = pscores[p];
    if (pclasses[p] != cls || !(s == s)) continue;          // uniform across the CTA
    const int img = pimages[p];
    Best mine{0.f, -1};
    for (int g = threadIdx.x; g < G; g += blockDim.x)
      if (!used[g] && tclasses[g] == cls && timages[g] == img) mine = better(mine, Best{box_iou_cxcywh(pboxes + 4 * p, tboxes + 4 * g), g});
    const Best win = block_argmax(mine, scratch);
    const bool hit = win.idx >= 0 && thr_ok && win.v >= thr;
    if (hit) { ++tp; if (threadIdx.x == 0) used[win.idx] = 1; } else { ++fp; }
    if (s >= score_thr) { if (hit) ++etp; else ++efp; }
    if (threadIdx.x == 0) {
      cv[2 * rank] = (float)tp / (float)(tp + fp);
      cv[2 * rank + 1] = targets ? (float)tp / (float)targets : 0.f;
    }
    ++rank;
    __syncthreads();
  }
  // 101-point interpolated AP: best precision among ranks whose recall reaches the required level
  __shared__ float ap_points[101];
  for (int rp = threadIdx.x; rp <= 100; rp += blockDim.x) {
    const float need = (float)rp * 0.01f;
    float best = 0.f;
    for (int r = 0; r < rank; ++r)
      if (cv[2 * r + 1] + 1e-7f >= need) best = fmaxf(best, cv[2 * r]);
    ap_points[rp] = best;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned fn = targets > etp ? targets - etp : 0u;
    counts[pair * 3 + 0] = etp; counts[pair * 3 + 1] = efp; counts[pair * 3 + 2] = fn;
    const float precision = etp + efp ? (float)etp / (float)(etp + efp) : 0.f, recall = targets ? (float)etp / (float)targets : 0.f;
    metrics[pair * 4 + 0] = precision; metrics[pair * 4 + 1] = recall;
    metrics[pair * 4 + 2] = precision + recall > 0.f ? 2.f * precision * recall / (precision + recall) : 0.f;
    float ap_sum = 0.f;
    for (int rp = 0; rp <= 100; ++rp) ap_sum += ap_points[rp];          // in order: reproducible
    metrics[pair * 4 + 3] = targets ? ap_sum / 101.f : 0.f;
  }
}

// One CTA: mAP per threshold over classes that have targets, and the mean over thresholds that had any such class
__global__ void detection_map_kernel(const unsigned* __restrict__ counts, const float* __restrict__ metrics, int thresholds, int classes,
                                     float* __restrict__ map_by_threshold, float* __restrict__ mean_map) {
  if (threadIdx.x != 0) return;
  float total = 0.f;
  int valid_t = 0;
  for (int t = 0; t < thresholds; ++t) {
    float sum = 0.f;
    int valid = 0;
    for (int c = 0; c < classes; ++c) {
      const int pair = t * classes + c;
      if (counts[pair * 3 + 0] + counts[pair * 3 + 2] == 0u) continue;
      sum += metrics[pair * 4 + 3];
      ++valid;
    }
    const float m = valid ? sum / (float)valid : 0.f;
    map_by_threshold[t] = m;
    if (valid) { total += m; ++valid_t; }
  }
  *mean_map = valid_t ? total / (float)valid_t : 0.f;
}

static inline int det_grid(long long n) {
  long long g = (n + 255) / 256;
  return (int)(g < 1 ? 1 : (g > 148 * 16 ? 148 * 16 : g));
}

}  // namespace oa

using namespace oa;

extern "C" {

int oa_det_box_iou(const void* a, const void* b, void* out, int n, int m, void* stream) {
  if (n <= 0 || m <= 0) return 0;
  box_iou_kernel<<<det_grid((long long)n * m), 256, 0, (cudaStream_t)stream>>>((const float*)a, (const float*)b, (float*)out, n, m);
  return (int)cudaGetLastError();
}

int oa_det_nms(const void* boxes, const void* scores, const void* classes, int n, float iou_thr, float score_thr, int max_det, int agnostic,
               void* indices, void* count, void* alive_scratch, void* stream) {
  nms_kernel<<<1, 1024, 0, (cudaStream_t)stream>>>((const float*)boxes, (const float*)scores, (const int*)classes, n, iou_thr, score_thr, max_det,
                                                    agnostic, (int*)indices, (unsigned*)count, (unsigned char*)alive_scratch);
  return (int)cudaGetLastError();
}

int oa_det_confusion(const void* predicted, const void* target, long long n, int classes, void* out_zeroed, void* stream) {
  if (n <= 0) return 0;
  confusion_kernel<<<det_grid(n), 256, 0, (cudaStream_t)stream>>>((const int*)predicted, (const int*)target, n, classes, (unsigned*)out_zeroed);
  return (int)cudaGetLastError();
}

int oa_det_binary_counts(const void* predicted, const void* target, long long n, void* out_zeroed, void* stream) {
  if (n <= 0) return 0;
  binary_counts_kernel<<<det_grid(n), 256, 0, (cudaStream_t)stream>>>((const unsigned char*)predicted, (const unsigned char*)target, n,
                                                                       (unsigned*)out_zeroed);
  return (int)cudaGetLastError();
}

int oa_det_segmentation_metrics(const void* confusion, int classes, void* per_class, void* mean_iou, void* accuracy, void* stream) {
  segmentation_metrics_kernel<<<1, 256, 0, (cudaStream_t)stream>>>((const unsigned*)confusion, classes, (float*)per_class, (float*)mean_iou,
                                                                   (float*)accuracy);
  return (int)cudaGetLastError();
}

int oa_det_evaluate(const void* pboxes, const void* pscores, const void* pclasses, const void* pimages, const void* order, int P,
                    const void* tboxes, const void* tclasses, const void* timages, int G, const void* thresholds, int T, int classes,
                    float score_thr, void* matched_scratch, void* curve_scratch, void* counts, void* metrics, void* map_by_threshold,
                    void* mean_map, void* stream) {
  if (T <= 0 || classes <= 0) return (int)cudaErrorInvalidValue;
  detection_curves_kernel<<<T * classes, 256, 0, (cudaStream_t)stream>>>(
      (const float*)pboxes, (const float*)pscores, (const int*)pclasses, (const int*)pimages, (const int*)order, P, (const float*)tboxes,
      (const int*)tclasses, (const int*)timages, G, (const float*)thresholds, classes, score_thr, (unsigned char*)matched_scratch,
      (float*)curve_scratch, (unsigned*)counts, (float*)metrics);
  detection_map_kernel<<<1, 32, 0, (cudaStream_t)stream>>>((const unsigned*)counts, (const float*)metrics, T, classes, (float*)map_by_threshold,
                                                           (float*)mean_map);
  return (int)cudaGetLastError();
}

}  // extern "C"
