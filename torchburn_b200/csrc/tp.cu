// Tensor-parallel exchange (placeholder until the communicator is wired in).
#include "tp.cuh"

namespace tb {

struct TpState { int dummy; };

tb_status tp_allreduce_residual(TpState* st, const float*, float*, int, int64_t, cudaStream_t, int*) {
  (void)st;
  return fail(TB_ERR_NCCL, "tensor-parallel decoder used before tb_decoder_tp_init");
}
tb_status tp_allgather_logits(TpState* st, const float*, float*, int, int64_t, cudaStream_t, int*) {
  (void)st;
  return fail(TB_ERR_NCCL, "tensor-parallel decoder used before tb_decoder_tp_init");
}
void tp_destroy(TpState* st) { delete st; }

}  // namespace tb

extern "C" {
tb_status tb_tp_unique_id(uint8_t id[128]) { (void)id; return tb::fail(TB_ERR_UNSUPPORTED, "tensor parallelism not built yet"); }
tb_status tb_decoder_tp_init(tb_decoder*, const uint8_t*, tb_allgather_fn, void*) {
  return tb::fail(TB_ERR_UNSUPPORTED, "tensor parallelism not built yet");
}
}
