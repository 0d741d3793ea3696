// Expert-parallel state behind a handle (ep.cu); used by the C ABI in api.cu.
#pragma once

#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

#include "../../include/dsmoe.h"

namespace dsmoe {

struct EpState;

int ep_get_unique_id(uint8_t *id128);
// id128: the 128-byte NCCL unique id every rank received from rank 0, or adopt_comm: an existing ncclComm_t.
int ep_create(const dsmoe_config &cfg, int device, const uint8_t *id128, void *adopt_comm, int rank, int world,
              uint32_t max_replicas, uint32_t recv_capacity_rows, EpState **out, char *err, size_t err_len);
void ep_destroy(EpState *s);
const char *ep_last_error(const EpState *s);
dsmoe_handle *ep_owner(EpState *s);
int ep_rank(const EpState *s);
int ep_world(const EpState *s);
int ep_p2p_combine(const EpState *s);  // 1: the combine is fused into the owner's down projection (peer stores)
int ep_set_replicas(EpState *s, uint32_t n_expert, const int32_t *ids, uint32_t n);
int ep_expert_counts(EpState *s, cudaStream_t st, uint32_t n_expert, uint64_t *host_out, int reset);
int ep_last_recv_rows(const EpState *s, int32_t *per_rank_out);
// marks: optional 6 events recorded at: start, plan done, dispatch done, owner compute done, combine done, sum done
int ep_forward(EpState *s, cudaStream_t st, uint32_t layer, const uint8_t *xq, const int32_t *selected, const float *weights,
               uint32_t n_tokens, uint32_t k, uint32_t n_embd, float *out, int *n_launched, cudaEvent_t *marks);

}  // namespace dsmoe
