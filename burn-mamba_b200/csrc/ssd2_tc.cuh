// Tensor-core (tcgen05 / TMEM / TMA) path of the Mamba-2 SSD forward.
#pragma once
#include "common.cuh"

namespace bm {
namespace tc {

// True when the tensor-core kernel covers this dtype/shape (bf16, headdim 64, state_rank 128, ...).
bool ssd2_supported(const bm_ssd2_fwd_args* a);
// Human-readable reason for ssd2_supported() == false.
const char* ssd2_why_not(const bm_ssd2_fwd_args* a);
size_t ssd2_workspace_bytes(const bm_ssd2_fwd_args* a);
int32_t ssd2_run(const bm_ssd2_fwd_args* a, void* workspace, size_t workspace_bytes, cudaStream_t stream);

// The same path with two heads of a B/C group per CTA (shared C/B loads and C B^T, 128-wide readout and
// state MMAs, sequence segments for load balance).  Needs an even number of heads per group.
bool ssd2_pair_supported(const bm_ssd2_fwd_args* a);
// True when the paired kernel is the better choice for this problem (more units than SMs).
bool ssd2_pair_preferred(const bm_ssd2_fwd_args* a);
size_t ssd2_pair_workspace_bytes(const bm_ssd2_fwd_args* a);
int32_t ssd2_pair_run(const bm_ssd2_fwd_args* a, void* workspace, size_t workspace_bytes, cudaStream_t stream);

// Mamba-2 SSD backward on the tensor cores (bf16, headdim 64, state_rank 128): a forward pass of the kernel
// above for the state entering every 128-token tile, then one reverse walk per (batch, head) unit.
bool ssd2_bwd_supported(const bm_ssd2_bwd_args* a);
const char* ssd2_bwd_why_not(const bm_ssd2_bwd_args* a);
size_t ssd2_bwd_workspace_bytes(const bm_ssd2_bwd_args* a);
int32_t ssd2_bwd_run(const bm_ssd2_bwd_args* a, void* workspace, size_t workspace_bytes, cudaStream_t stream);

// The Mamba-3 cores (single-pass with gamma / scale, or the generic core) on the one-head-per-CTA kernel, over the
// fused (time x rank) axis.  bf16, headdim 64, state_rank 128, MIMO rank 1, 2 or 4.  When `angles` is given, B and C
// are rotated inside the kernel, on the tiles in shared memory.
bool ssd3_supported(const bm_ssd3_fwd_args* a);
const char* ssd3_why_not(const bm_ssd3_fwd_args* a);
size_t ssd3_workspace_bytes(const bm_ssd3_fwd_args* a);
// chunk_states (optional, internal): [b, tiles, h, p, r] float32, the state entering every 128-row tile.
int32_t ssd3_run(const bm_ssd3_fwd_args* a, bool single, void* workspace, size_t workspace_bytes, cudaStream_t stream,
                 float* chunk_states = nullptr);

// Backward of the Mamba-3 cores on the tensor cores (same kernel as the Mamba-2 backward, on the fused axis).
bool ssd3_bwd_supported(const bm_ssd3_bwd_args* a);
const char* ssd3_bwd_why_not(const bm_ssd3_bwd_args* a);
size_t ssd3_bwd_workspace_bytes(const bm_ssd3_bwd_args* a);
int32_t ssd3_bwd_run(const bm_ssd3_bwd_args* a, bool single, void* workspace, size_t workspace_bytes, cudaStream_t stream);

}  // namespace tc
}  // namespace bm
