// Host side of TMA: builds CUtensorMap descriptors for (B,H,L,D) views.  The driver entry point is
// looked up through the runtime so the library does not link against libcuda.
#include <cudaTypedefs.h>

#include <mutex>

#include "jvpattn_common.cuh"
#include "sm100_ptx.cuh"

namespace jvpattn {
namespace {

PFN_cuTensorMapEncodeTiled_v12000 g_encode = nullptr;
std::once_flag g_encode_once;

void resolve_encode() {
  void *fn = nullptr;
  cudaDriverEntryPointQueryResult qres;
  cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres);
  if (e == cudaSuccess && qres == cudaDriverEntryPointSuccess) g_encode = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(fn);
  (void)cudaGetLastError();
}

}  // namespace

bool make_tensor_map(CUtensorMap *out, const void *ptr, int dtype, int B, int H, int L, int D, int64_t sb, int64_t sh,
                     int64_t sl, int box_rows) {
  std::call_once(g_encode_once, resolve_encode);
  if (!g_encode) return false;
  if (reinterpret_cast<uintptr_t>(ptr) % 16 != 0) return false;
  if (D % 64 != 0 || box_rows < 1 || box_rows > 256) return false;
  const cuuint64_t dims[4] = {(cuuint64_t)D, (cuuint64_t)L, (cuuint64_t)H, (cuuint64_t)B};
  // a size-1 axis may carry a meaningless stride; any multiple of 16 bytes will do for it
  auto fix = [&](int64_t s, int n) -> int64_t { return n == 1 ? (int64_t)D : s; };
  const int64_t es[3] = {fix(sl, L), fix(sh, H), fix(sb, B)};
  cuuint64_t strides[3];
  for (int i = 0; i < 3; ++i) {
    if (es[i] <= 0 || (es[i] * 2) % 16 != 0) return false;
    strides[i] = (cuuint64_t)es[i] * 2;
  }
  const cuuint32_t box[4] = {64, (cuuint32_t)box_rows, 1, 1};
  const cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = g_encode(out, dtype == JVPATTN_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4,
                        const_cast<void *>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                        CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

}  // namespace jvpattn
