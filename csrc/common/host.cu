#include "host.hpp"

#include <mutex>

namespace bb {

EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) ==
            cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}

int make_tmap_2d(CUtensorMap* out, CUtensorMapDataType dt, int elem_size, const void* base,
                 uint64_t inner, uint64_t outer, uint64_t row_stride_bytes, uint32_t box_inner,
                 uint32_t box_outer, bool swizzle128) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return BB_EDRIVER;
  if ((reinterpret_cast<uintptr_t>(base) & 15) || (row_stride_bytes & 15)) return BB_EARG;
  cuuint64_t dims[2] = {inner, outer};
  cuuint64_t strides[1] = {row_stride_bytes};
  cuuint32_t box[2] = {box_inner, box_outer};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = CUDA_SUCCESS;
  for (int attempt = 0; attempt < 2; ++attempt) {
    r = fn(out, dt, 2, const_cast<void*>(base), dims, strides, box, estr,
           CU_TENSOR_MAP_INTERLEAVE_NONE,
           swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
           CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r == CUDA_SUCCESS) break;
    cudaFree(0);  // a worker thread (e.g. autograd's) may not have the primary context bound yet
  }
  (void)elem_size;
  return r == CUDA_SUCCESS ? BB_OK : -(1000 + (int)r);
}

int make_tmap_3d(CUtensorMap* out, CUtensorMapDataType dt, int elem_size, const void* base,
                 uint64_t d0, uint64_t d1, uint64_t d2, uint64_t s1_bytes, uint64_t s2_bytes,
                 uint32_t box0, uint32_t box1, bool swizzle128) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return BB_EDRIVER;
  if ((reinterpret_cast<uintptr_t>(base) & 15) || (s1_bytes & 15) || (s2_bytes & 15))
    return BB_EARG;
  cuuint64_t dims[3] = {d0, d1, d2};
  cuuint64_t strides[2] = {s1_bytes, s2_bytes};
  cuuint32_t box[3] = {box0, box1, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = CUDA_SUCCESS;
  for (int attempt = 0; attempt < 2; ++attempt) {
    r = fn(out, dt, 3, const_cast<void*>(base), dims, strides, box, estr,
           CU_TENSOR_MAP_INTERLEAVE_NONE,
           swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
           CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r == CUDA_SUCCESS) break;
    cudaFree(0);  // a worker thread (e.g. autograd's) may not have the primary context bound yet
  }
  (void)elem_size;
  return r == CUDA_SUCCESS ? BB_OK : -(1000 + (int)r);
}

__device__ int g_error_word[4];

int* device_error_word() {
  static int* ptrs[64] = {nullptr};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) return nullptr;
  if (!ptrs[dev]) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_error_word) != cudaSuccess) return nullptr;
    ptrs[dev] = static_cast<int*>(p);
  }
  return ptrs[dev];
}

int sm_count() {
  static int counts[64] = {0};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) return 148;
  if (!counts[dev]) {
    int n = 0;
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    counts[dev] = n > 0 ? n : 148;
  }
  return counts[dev];
}

}  // namespace bb

// Read-and-clear the device error word (synchronises the device). 0 = no kernel reported a timeout.
BB_API int bb_read_error(int clear) {
  int* w = bb::device_error_word();
  if (!w) return -1;
  int v = 0;
  if (cudaMemcpy(&v, w, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return -2;
  if (clear && v != 0) cudaMemset(w, 0, sizeof(int));
  return v;
}

// Non-blocking check of the device error word: each call first harvests the copy that the previous
// call enqueued (if it has completed) and then enqueues a new async copy of the word into pinned host
// memory on `stream`.  Returns the last harvested value (0 = clean, >0 = a kernel's bounded wait ran
// out), -1 on a set-up failure.  The answer therefore trails the kernels by one call; the caller
// makes one call per step.  A non-zero value is sticky until bb_read_error(1) clears the word.
BB_API int bb_poll_error(void* stream) {
  struct Slot { int* host = nullptr; cudaEvent_t ev = nullptr; bool pending = false; int last = 0; };
  static Slot slots[64];
  static std::mutex mu;
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) return -1;
  int* w = bb::device_error_word();
  if (!w) return -1;
  std::lock_guard<std::mutex> lk(mu);
  Slot& s = slots[dev];
  if (!s.host) {
    if (cudaHostAlloc(reinterpret_cast<void**>(&s.host), sizeof(int), cudaHostAllocDefault) != cudaSuccess)
      return -1;
    *s.host = 0;
    if (cudaEventCreateWithFlags(&s.ev, cudaEventDisableTiming) != cudaSuccess) return -1;
  }
  if (s.pending) {
    if (cudaEventQuery(s.ev) != cudaSuccess) return s.last;  // still in flight: keep the older answer
    s.last = *s.host;
    s.pending = false;
  }
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (cudaMemcpyAsync(s.host, w, sizeof(int), cudaMemcpyDeviceToHost, st) == cudaSuccess &&
      cudaEventRecord(s.ev, st) == cudaSuccess)
    s.pending = true;
  return s.last;
}

BB_API int bb_sm_count() { return bb::sm_count(); }
