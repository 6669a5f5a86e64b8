// Helpers of the slab mode (a grid split along K across GPUs; gridnet_b200/slab.py).
#include "common.cuh"
#include "kernels.h"

namespace gn {

// x[b][m][n][col_left] = from_left[b][m][n] and x[b][m][n][col_right] = from_right[b][m][n]: the
// neighbours' boundary faces, delivered packed, go into the ghost columns the step kernel reads
// as halo cells. Either source may be null (end of the grid).
__global__ void __launch_bounds__(256) slab_unpack_faces_k(const float *__restrict__ from_left,
                                                           const float *__restrict__ from_right, float *__restrict__ x,
                                                           size_t cells, int K, int col_left, int col_right)
{
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= cells) return;
    if (from_left) x[i * K + col_left] = from_left[i];
    if (from_right) x[i * K + col_right] = from_right[i];
}

int launch_slab_unpack_faces(const float *from_left, const float *from_right, float *x, int B, int M, int N, int K,
                             int col_left, int col_right, cudaStream_t st)
{
    const size_t cells = (size_t)B * M * N;
    if (cells == 0 || (!from_left && !from_right)) return GN_OK;
    slab_unpack_faces_k<<<(unsigned)((cells + 255) / 256), 256, 0, st>>>(from_left, from_right, x, cells, K, col_left,
                                                                        col_right);
    return check_launch("slab_unpack_faces");
}

}  // namespace gn
