// Tensor-parallel exchange steps of the decoder (see tp.cu).
#pragma once
#include "tb_common.cuh"

namespace tb {

struct TpState;

// x[b, :] += sum over ranks of partial[b, :]   (after a row-parallel projection)
tb_status tp_allreduce_residual(TpState* st, const float* partial, float* x, int batch, int64_t hidden,
                                cudaStream_t stream, int* launches);
// logits[b, r*V_l : (r+1)*V_l] = rank r's logits_l[b, :]
tb_status tp_allgather_logits(TpState* st, const float* logits_l, float* logits, int batch,
                              int64_t v_local, cudaStream_t stream, int* launches);
void tp_destroy(TpState* st);

}  // namespace tb
