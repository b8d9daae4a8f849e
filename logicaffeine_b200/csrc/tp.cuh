// Tensor-parallel group: NCCL communicator resolved at run time (tp.cu).
#pragma once
#include <nccl.h>
#include <string.h>

#include "common.cuh"

namespace logos {

struct TpGroup {
  int   degree = 1;
  int   rank = 0;
  void* comm = nullptr;  // ncclComm_t
};

logos_status_t tp_unique_id(void* out_128);
logos_status_t tp_init(TpGroup* g, int degree, int rank, const void* unique_id_128);
void tp_destroy(TpGroup* g);
// In-place sum over the group; every rank ends with identical bits.
logos_status_t tp_allreduce_sum_f32(TpGroup* g, float* buf, int64_t count, cudaStream_t st);
logos_status_t tp_allgather_bytes(TpGroup* g, const void* send, void* recv, int64_t bytes_per_rank, cudaStream_t st);

}  // namespace logos
