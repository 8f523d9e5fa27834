// Host-side construction of TMA tensor maps (cuTensorMapEncodeTiled through the runtime's
// driver entry point lookup; no direct libcuda link).
#include <mutex>

#include "common.cuh"
#include "sm100_ptx.cuh"

namespace alg {

EncodeTiledFn get_encode_tiled() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}

int make_tmap_bf16(CUtensorMap* out, const void* base, int rank, const uint64_t* dims, const uint64_t* strides_elems,
                   const uint32_t* box, bool swizzle128) {
  EncodeTiledFn enc = get_encode_tiled();
  if (enc == nullptr) {
    set_error("cuTensorMapEncodeTiled is not available from this driver");
    return ALG_ERR_CUDA;
  }
  cuuint64_t gdim[5], gstride[4];
  cuuint32_t bdim[5], estride[5];
  for (int i = 0; i < rank; ++i) {
    gdim[i] = dims[i];
    bdim[i] = box[i];
    estride[i] = 1;
    if (i > 0) {
      gstride[i - 1] = strides_elems[i - 1] * 2;          // bytes
      if (gstride[i - 1] % 16 != 0) {
        set_error("TMA needs strides that are multiples of 16 bytes (dim %d stride %llu B)", i,
                  (unsigned long long)gstride[i - 1]);
        return ALG_ERR_INVALID;
      }
    }
  }
  if ((reinterpret_cast<uintptr_t>(base) & 15) != 0) {
    set_error("TMA needs a 16-byte aligned base address");
    return ALG_ERR_INVALID;
  }
  CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, cuuint32_t(rank), const_cast<void*>(base), gdim, gstride,
                   bdim, estride, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_error("cuTensorMapEncodeTiled failed with CUresult %d", int(r));
    return ALG_ERR_CUDA;
  }
  return ALG_OK;
}

}  // namespace alg
