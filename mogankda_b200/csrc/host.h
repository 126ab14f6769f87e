// Host-side helpers shared by the launchers: error text behind mkda_last_error() and launch checking.
#pragma once
#include <stdint.h>
#include <cuda.h>
#include <cuda_runtime.h>

#include "../../include/mkda.h"

namespace mkda {
int set_error(int code, const char* msg);
int check_launch(const char* what);
// Raises the dynamic shared memory limit of `func` (the attribute is set once per function and device; later calls
// return at once); returns 0 or an error code.
int ensure_smem(const void* func, int bytes, const char* what);
// Tensor map over a row-major [rows][row_elems] tensor of 2- or 4-byte elements whose boxes are 64 rows x 128 elements, not
// swizzled: one tiled TMA copy then brings 64 strided 128-element rows (token rows of one head) into shared memory as a dense
// [64][128] block.  Rows past the end of the tensor read as zeros.  Returns 0, or an error code when the tensor cannot be
// described (base not 16-byte aligned, row pitch not a multiple of 16 bytes, or the driver lacks the encoder).
int make_rows_map(CUtensorMap* out, const void* base, int elem_bytes, unsigned long long rows, unsigned long long row_elems, const char* what);
// True if any of the (possibly null) pointers is not 16-byte aligned: the kernels read and write their tensors with
// 16-byte vector accesses and bulk copies, and a misaligned address would fault the device instead of returning an error.
template <typename... P>
inline bool any_misaligned(P... ptrs) {
    return (((reinterpret_cast<uintptr_t>(static_cast<const void*>(ptrs)) & 15) != 0) || ...);
}
// Number of SMs of the current device (cached per device).
int sm_count();
int launch_out_fwd_tc(const MkdaOutFwd* p, cudaStream_t stream);
int tc_chunk_status(unsigned int* out);
int tc_chunk_status_clear();
int launch_recur_fwd_tc(const MkdaRecurFwd* p, cudaStream_t stream);
int launch_bwd_dh_tc(const MkdaBwdDh* p, cudaStream_t stream);
int tc_recur_status(unsigned int* out);
int tc_recur_status_clear();
int launch_intra_fwd_tc(const MkdaIntraFwd* p, cudaStream_t stream);
int launch_bwd_chunk_tc(const MkdaBwdChunk* p, cudaStream_t stream);
int tc_intra_status(unsigned int* out);
int tc_intra_status_clear();
}  // namespace mkda
