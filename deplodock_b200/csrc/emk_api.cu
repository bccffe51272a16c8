// Handle lifetime, status plumbing and the host-side TMA tensor-map encoder of the emk library.
// The reference reaches cuTensorMapEncodeTiled through ctypes on libcuda (emmy/compiler/backend/cuda/_tma.py:66-170);
// here the driver entry point is resolved once per handle with cudaGetDriverEntryPoint, so the library needs no link
// against libcuda and loads on a machine without a driver.
#include "emk_common.cuh"

#include <stdlib.h>

extern "C" int emk_version(void) { return EMK_VERSION; }

extern "C" int emk_bounds_check_enabled(void) {
#ifdef EMK_BOUNDS_CHECK
  return 1;
#else
  return 0;
#endif
}

extern "C" const char* emk_status_string(int s) {
  switch (s) {
    case EMK_OK: return "ok";
    case EMK_ERR_SHAPE: return "unsupported or invalid shape";
    case EMK_ERR_DTYPE: return "unsupported dtype";
    case EMK_ERR_ALIGN: return "pointer or leading dimension misaligned";
    case EMK_ERR_WORKSPACE: return "workspace too small";
    case EMK_ERR_CUDA: return "CUDA call failed";
    case EMK_ERR_TIMEOUT: return "device-side wait expired";
    case EMK_ERR_ARG: return "invalid argument";
    case EMK_ERR_LIMIT: return "size beyond the entry point's fixed maximum";
    case EMK_ERR_BOUNDS: return "a data-dependent index was out of range (bounds-check build)";
    default: return "unknown status";
  }
}

extern "C" int emk_create(int device, emk_handle_t* out) {
  if (!out) return EMK_ERR_ARG;
  *out = nullptr;
  if (device < 0 || device >= EMK_MAX_DEVICES) return EMK_ERR_ARG;
  int caller_device = -1;
  if (cudaGetDevice(&caller_device) != cudaSuccess) caller_device = -1;
  // the handle's set-up runs with `device` current; the caller's current device is put back on every way out
  struct Restore {
    int dev;
    ~Restore() {
      if (dev >= 0) (void)cudaSetDevice(dev);
    }
  } restore{caller_device == device ? -1 : caller_device};
  emk_handle_s* h = (emk_handle_s*)calloc(1, sizeof(emk_handle_s));
  if (!h) return EMK_ERR_ARG;
  h->device = device;
  h->wait_limit_ns = 2000ull * 1000ull * 1000ull;
  const char* impl = getenv("EMK_GEMM_IMPL");
  h->gemm_impl = impl ? atoi(impl) : 0;
  const char* ovl = getenv("EMK_OVERLAP_LAUNCH");
  h->overlap_launch = (ovl && atoi(ovl) == 0) ? 0 : 1;
  const char* cgm = getenv("EMK_CHAIN_GROUP_M");
  h->chain_group_m = (cgm && atoi(cgm) > 0) ? atoi(cgm) : 2;
  cudaError_t e = cudaSetDevice(device);
  if (e != cudaSuccess) {
    free(h);
    return EMK_ERR_CUDA;
  }
  cudaDeviceProp prop;
  e = cudaGetDeviceProperties(&prop, device);
  if (e != cudaSuccess) {
    free(h);
    return EMK_ERR_CUDA;
  }
  h->sm_count = prop.multiProcessorCount;
  h->max_smem_optin = (int)prop.sharedMemPerBlockOptin;
  void* fn = nullptr;
  cudaDriverEntryPointQueryResult qres;
  e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres);
  if (e != cudaSuccess || qres != cudaDriverEntryPointSuccess || !fn) {
    free(h);
    return EMK_ERR_CUDA;
  }
  h->encode_tiled = (emk_encode_tiled_fn)fn;
  e = cudaHostAlloc((void**)&h->status_host, 64, cudaHostAllocMapped);
  if (e != cudaSuccess) {
    free(h);
    return EMK_ERR_CUDA;
  }
  h->status_host[0] = 0;
  e = cudaHostGetDevicePointer((void**)&h->status_dev, h->status_host, 0);
  if (e != cudaSuccess) {
    cudaFreeHost(h->status_host);
    free(h);
    return EMK_ERR_CUDA;
  }
  *out = h;
  return EMK_OK;
}

extern "C" int emk_destroy(emk_handle_t h) {
  if (!h) return EMK_ERR_ARG;
  if (h->status_host) cudaFreeHost(h->status_host);
  free(h);
  return EMK_OK;
}

extern "C" const char* emk_last_error(emk_handle_t h) { return h ? h->last_error : "null handle"; }

extern "C" int emk_set_wait_limit_ms(emk_handle_t h, int ms) {
  if (!h || ms <= 0) return EMK_ERR_ARG;
  h->wait_limit_ns = (unsigned long long)ms * 1000000ull;
  return EMK_OK;
}

extern "C" int emk_set_launch_overlap(emk_handle_t h, int on) {
  if (!h) return -EMK_ERR_ARG;
  const int prev = h->overlap_launch;
  h->overlap_launch = on ? 1 : 0;
  return prev;
}

extern "C" int emk_device_status(emk_handle_t h, emk_stream_t stream) {
  if (!h) return EMK_ERR_ARG;
  EMK_CUDA_TRY(h, cudaStreamSynchronize((cudaStream_t)stream));
  int code = *(volatile int*)h->status_host;
  if (code != 0) {
    *(volatile int*)h->status_host = 0;
    if (code >= EMK_DEV_BOUNDS_TOKEN_ID) {
      EMK_SET_ERR(h, "out-of-range %s (code %d); the access was clamped or dropped",
                  code == EMK_DEV_BOUNDS_TOKEN_ID ? "token id in the embedding gather"
                  : code == EMK_DEV_BOUNDS_POSITION ? "rotary position"
                  : "sequence in cu_seqlens", code);
      return EMK_ERR_BOUNDS;
    }
    EMK_SET_ERR(h, "device-side wait expired (role code %d)", code);
    return EMK_ERR_TIMEOUT;
  }
  EMK_CUDA_TRY(h, cudaGetLastError());
  return EMK_OK;
}

int emk_make_tmap_2d(emk_handle_t h, CUtensorMap* out, CUtensorMapDataType dt, int elem_bytes, const void* base,
                     uint64_t inner, uint64_t outer, uint64_t pitch_bytes, uint32_t box_inner, uint32_t box_outer,
                     CUtensorMapSwizzle swizzle) {
  if (((uintptr_t)base & 15u) != 0 || (pitch_bytes & 15u) != 0) {
    EMK_SET_ERR(h, "tensor map operand must be 16-byte aligned with a 16-byte multiple row pitch");
    return EMK_ERR_ALIGN;
  }
  cuuint64_t dims[2] = {inner, outer};
  cuuint64_t strides[1] = {pitch_bytes};
  cuuint32_t box[2] = {box_inner, box_outer};
  cuuint32_t estr[2] = {1, 1};
  (void)elem_bytes;
  CUresult r = h->encode_tiled(out, dt, 2, const_cast<void*>(base), dims, strides, box, estr,
                               CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    EMK_SET_ERR(h, "cuTensorMapEncodeTiled failed with CUresult %d (inner=%llu outer=%llu pitch=%llu box=%ux%u)",
                (int)r, (unsigned long long)inner, (unsigned long long)outer, (unsigned long long)pitch_bytes,
                box_inner, box_outer);
    return EMK_ERR_CUDA;
  }
  return EMK_OK;
}

// ---------------------------------------------------------------------------------------------------------------
// Bounded-wait self test: one warp waits on a barrier that never completes, gives up after the limit, records the
// expiry and returns. The kernel always terminates.
// ---------------------------------------------------------------------------------------------------------------
__global__ void emk_wait_expiry_kernel(int* status, unsigned long long limit_ns) {
  __shared__ uint64_t bar;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    abort_flag = 0;
    emk::mbar_init(&bar, 1);
    emk::fence_barrier_init();
  }
  __syncthreads();
  emk::WaitCtx w{&abort_flag, status, limit_ns};
  if (threadIdx.x == 0) {
    emk::mbar_wait(&bar, 0, w, EMK_DEV_TIMEOUT_SELFTEST);
  }
  __syncthreads();
}

extern "C" int emk_selftest_wait_expiry(emk_handle_t h, int limit_ms, emk_stream_t stream) {
  if (!h || limit_ms <= 0 || limit_ms > 1000) return EMK_ERR_ARG;
  emk_wait_expiry_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(h->status_dev, (unsigned long long)limit_ms * 1000000ull);
  EMK_LAUNCH_CHECK(h);
  return EMK_OK;
}
