// ls100_ctx: device bookkeeping shared by every kernel family.
#include "ctx.h"

#include <stdio.h>
#include <stdlib.h>

int ls100_gemm_i8_init_device();
int ls100_attn_init_device();
int ls100_proj_tc_init_device();

bool ls100_pdl_enabled() {
  static const bool on = [] {
    const char* e = getenv("LS100_PDL");
    return !(e && e[0] == '0');
  }();
  return on;
}

extern "C" int ls100_ctx_create(ls100_ctx** out, int device) {
  if (!out) return LS100_ERR_BAD_ARG;
  *out = nullptr;
  if (cudaSetDevice(device) != cudaSuccess) return LS100_ERR_CUDA;
  cudaDeviceProp prop;
  if (cudaGetDeviceProperties(&prop, device) != cudaSuccess) return LS100_ERR_CUDA;
  if (prop.major != 10) {
    fprintf(stderr, "ls100: device %d is sm_%d%d; this library only runs on sm_100a (B200)\n", device, prop.major,
            prop.minor);
    return LS100_ERR_UNSUPPORTED;
  }
  ls100_ctx* c = new ls100_ctx();
  c->device = device;
  c->sm_count = prop.multiProcessorCount;
  if (cudaMalloc(&c->d_err, sizeof(int)) != cudaSuccess || cudaMemset(c->d_err, 0, sizeof(int)) != cudaSuccess) {
    delete c;
    return LS100_ERR_CUDA;
  }
  void* fn = nullptr;
  cudaDriverEntryPointQueryResult qres;
  if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres) != cudaSuccess ||
      qres != cudaDriverEntryPointSuccess || !fn) {
    cudaFree(c->d_err);
    delete c;
    return LS100_ERR_NO_DRIVER;
  }
  c->encode = (ls100_encode_tiled_fn)fn;
  if (ls100_gemm_i8_init_device() != LS100_OK || ls100_attn_init_device() != LS100_OK ||
      ls100_proj_tc_init_device() != LS100_OK) {
    cudaFree(c->d_err);
    delete c;
    return LS100_ERR_CUDA;
  }
  *out = c;
  return LS100_OK;
}

extern "C" void ls100_ctx_destroy(ls100_ctx* ctx) {
  if (!ctx) return;
  cudaSetDevice(ctx->device);
  cudaFree(ctx->d_err);
  delete ctx;
}

extern "C" const char* ls100_strerror(int code) {
  switch (code) {
    case LS100_OK: return "ok";
    case LS100_ERR_BAD_ARG: return "bad argument (null pointer or non-positive size)";
    case LS100_ERR_ALIGN: return "pointer or leading dimension not 16-byte aligned";
    case LS100_ERR_UNSUPPORTED: return "unsupported shape or device";
    case LS100_ERR_CUDA: return "CUDA call failed";
    case LS100_ERR_TIMEOUT: return "a bounded device-side wait gave up";
    case LS100_ERR_NO_DRIVER: return "cuTensorMapEncodeTiled entry point unavailable";
    default: return "unknown ls100 error";
  }
}

extern "C" int ls100_ctx_poll_error(ls100_ctx* ctx, ls100_stream_t stream) {
  if (!ctx) return LS100_ERR_BAD_ARG;
  if (cudaStreamSynchronize((cudaStream_t)stream) != cudaSuccess) return LS100_ERR_CUDA;
  int h = 0;
  if (cudaMemcpy(&h, ctx->d_err, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return LS100_ERR_CUDA;
  if (h != 0) cudaMemset(ctx->d_err, 0, sizeof(int));
  return h;
}

extern "C" int ls100_sm_count(const ls100_ctx* ctx) { return ctx ? ctx->sm_count : 0; }

int ls100_get_tmap_u8(ls100_ctx* ctx, const void* ptr, uint64_t rows, uint64_t cols, uint64_t ld_bytes,
                      uint32_t box_rows, uint32_t box_cols, CUtensorMap* out) {
  ls100_tmap_key key{ptr, rows, cols, ld_bytes, box_rows, box_cols};
  std::lock_guard<std::mutex> lk(ctx->mu);
  auto it = ctx->tmaps.find(key);
  if (it != ctx->tmaps.end()) {
    *out = it->second;
    return LS100_OK;
  }
  CUtensorMap tm;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {ld_bytes};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = ctx->encode(&tm, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                           CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return LS100_ERR_CUDA;
  if (ctx->tmaps.size() > 4096) ctx->tmaps.clear();
  ctx->tmaps.emplace(key, tm);
  *out = tm;
  return LS100_OK;
}
