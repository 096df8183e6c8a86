/* bobcat-cuda: diagnostics for this library's own tests and benchmark.
 *
 * None of these has a counterpart a bobcat binding would call: the reference reads its runner's
 * state directly in Rust tests (crates/bobcat/tests/lfm2_reference.rs:118-151) and computes its
 * roofline bytes in the benchmark binary (crates/bobcat-bench/src/bin/bobcat_bench.rs). They are
 * exported from the same shared library so the parity tests can look inside a sequence, but they
 * are not part of the drop-in boundary declared in bobcat_cuda.h. */
#ifndef BOBCAT_CUDA_TEST_H
#define BOBCAT_CUDA_TEST_H

#include "bobcat_cuda.h"

#ifdef __cplusplus
extern "C" {
#endif

/* Bytes of weights one decoded token reads (every matrix once, active experts only), the figure
 * the decode roofline divides by (docs/design.md:15-34). */
uint64_t bc_model_decode_bytes(const bc_model* model);
/* Read back sequence state: which = 0 conv / DeltaNet conv history, 1 K cache, 2 V cache (as
 * f32), 3 DeltaNet state, 4 the routes the last traced pass of a mixture-of-experts model recorded
 * ([layer][trace row][2 * n_used] 32-bit words, the word bits in the floats; one trace row after a
 * traced step, the prefill batch size after a traced prefill). `layer` indexes layers of that kind. Returns the float count in `n` and
 * fills `out` (capacity `cap` floats) when non-null. */
bc_status bc_seq_read_state(bc_seq* seq, int32_t which, uint32_t layer, float* out, size_t cap, size_t* n);
/* Timing diagnostics: leave every launch called `name` (of n_rows x n_cols when those are nonzero)
 * out of this sequence's forward passes, so the time one kind of launch costs inside a replayed
 * decode step is the difference against a full step. The passes then compute garbage; NULL or ""
 * restores them. */
bc_status bc_seq_set_skip(bc_seq* seq, const char* name, uint32_t n_rows, uint32_t n_cols);
/* How many kernels this sequence has launched so far (its own kernels, not library calls). */
uint64_t bc_seq_launches(const bc_seq* seq);

#ifdef __cplusplus
}
#endif
#endif /* BOBCAT_CUDA_TEST_H */
