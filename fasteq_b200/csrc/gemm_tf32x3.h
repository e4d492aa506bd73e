// Interface between the SO3Linear entry points and the tensor-core grouped GEMM.
#pragma once
#include <cstdint>
#include <cuda.h>
#include <cuda_runtime.h>
namespace fasteq {
namespace tc {
struct TcTable {
  int n_groups, n_items;       // an item is one (group, row t) pair = one output row block
  int group_c_row[64];         // first output row of the group
  int group_first[65];         // segments (paths) of group g: [first[g], first[g+1])
  int item_first[65];          // items of group g: [item_first[g], item_first[g+1])
  int path_a_row[64];          // first row of A the segment reads
  int path_w[64];              // block of Bt the segment multiplies with
};
bool supported(long long M, int a_rows, int K, int P, int N, int c_rows, const void* A, const void* Bt, const void* C);
int launch(const TcTable& tab, const float* A, long long M, int a_rows, int K, const float* Bt_hi, const float* Bt_lo, int P, int N,
           float* C, int c_rows, cudaStream_t s);
int device_status(int* code);
// 3-D FP32 tensor [d2][d1][d0] (d0 contiguous, strides in elements), box [b2][b1][b0], SWIZZLE_128B, zero fill
int make_map(CUtensorMap* m, const float* base, uint64_t d0, uint64_t d1, uint64_t d2, uint64_t stride1_elems,
             uint64_t stride2_elems, uint32_t b0, uint32_t b1, uint32_t b2);
}  // namespace tc
namespace chain {
int device_status(int* code);   // status word of the radial-chain kernels (read and cleared)
}  // namespace chain
}  // namespace fasteq
