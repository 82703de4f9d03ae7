// tcgen05 (5th-generation tensor core) kernels: placeholder while the CUDA-core path is validated.
#include "common.cuh"
namespace b200 {
bool tc_supported(const ConvGeom&, int) { return false; }
size_t tc_workspace(const ConvGeom&, int, size_t, int*, int*) { return 0; }
int tc_forward(const ConvGeom&, View4, View4, const float*, long long, float*, void*, size_t, cudaStream_t) { return fail(B200_EUNSUPPORTED, "tcgen05 path not built"); }
int tc_dinput(const ConvGeom&, View4, View4, float*, void*, size_t, cudaStream_t) { return fail(B200_EUNSUPPORTED, "tcgen05 path not built"); }
int tc_dweight(const ConvGeom&, View4, View4, float*, void*, size_t, cudaStream_t) { return fail(B200_EUNSUPPORTED, "tcgen05 path not built"); }
int tc_gemm(long long, long long, long long, const float*, long long, long long, const float*, long long, long long, const float*, float, float, float*, cudaStream_t) { return B200_EUNSUPPORTED; }
}
