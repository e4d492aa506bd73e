// Interface between the SO3Linear entry points and the tensor-core grouped GEMM.
#pragma once
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
int launch(const TcTable& tab, const float* A, long long M, int a_rows, int K, const float* Bt, int P, int N, float* C,
           int c_rows, cudaStream_t s);
int device_status(int* code);
}  // namespace tc
}  // namespace fasteq
