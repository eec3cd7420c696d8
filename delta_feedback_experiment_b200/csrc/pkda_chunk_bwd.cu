// placeholder until the backward kernels land
#include "pkda_chunk.cuh"
namespace pkda {
size_t chunk_bwd_workspace(const pkda_problem& p) { return 0; }
int chunk_bwd(const pkda_chunk_bwd_args* a, cudaStream_t st) { return PKDA_ERR_SHAPE; }
}
