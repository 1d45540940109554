// Tensor-parallel exchange steps of the decoder (see tp.cu).
#pragma once
#include "tb_common.cuh"

namespace tb {

struct TpState;

// x[b, :] += sum over ranks of partial[b, :]   (after a row-parallel projection)
// With scale_w / out_scaled / out_ss8 (low-latency exchange only, see tp_low_latency) the kernel also
// writes x * scale_w and the sums of squares of x per 8 elements: the split RMSNorm of the decoder.
tb_status tp_allreduce_residual(TpState* st, const float* partial, float* x, int batch, int64_t hidden,
                                cudaStream_t stream, int* launches, const float* scale_w = nullptr,
                                float* out_scaled = nullptr, float* out_ss8 = nullptr);
// True when an exchange of this size takes the low-latency form (small, peer memory available).
bool tp_low_latency(const TpState* st, int batch, int64_t hidden);
// logits[b, r*V_l : (r+1)*V_l] = rank r's logits_l[b, :]
tb_status tp_allgather_logits(TpState* st, const float* logits_l, float* logits, int batch,
                              int64_t v_local, cudaStream_t stream, int* launches);
void tp_destroy(TpState* st);
// Communicator (NCCL) and, when `allgather` is given and nccl_only is false, the peer-memory
// exchange buffers.  Collective: every rank calls it.  max_count = floats per partial.
// hidden / logit_floats size the areas of the persistent step kernel (0: none).
tb_status tp_create(TpState** out, int rank, int size, const uint8_t id[128], size_t max_count,
                    tb_allgather_fn allgather, void* user, bool nccl_only, size_t hidden = 0, size_t logit_floats = 0);
// Fills `t` with the peer-visible areas of the step kernel; false when there are none.
bool tp_step_areas(TpState* st, StepTp* t);
// This rank's copy of the gathered logits inside the shared block (null when there is none).
float* tp_step_logits(TpState* st);
// Where the row-parallel projection of the NEXT tp_allreduce_residual call must write its
// partial (the peer-visible buffer on the fused path, `fallback` otherwise).
float* tp_partial_buffer(TpState* st, float* fallback);
// 1 after a bounded wait on a peer ran out.
int tp_error_flag(TpState* st);
// The exchange kernels also raise this host-mapped word (device pointer) when a bounded wait runs out.
void tp_set_host_fault(TpState* st, int* device_pointer_of_mapped_word);
// Test hook: limit in clock cycles of the exchange kernels' waits for their peers (0 = default, ~10 s).
void tp_set_wait_limit(long long cycles);

}  // namespace tb
