/* libbobcat_synth: writes synthetic GGUF model files for the tests and the benchmark.
 *
 * No reference counterpart: the reference only reads GGUF (crates/bobcat-gguf/src/lib.rs) and
 * measures on downloaded checkpoints. Files written here follow the layout that parser checks
 * (magic, version 3, general.alignment, aligned tensor offsets, whole quant blocks per row).
 * This is test infrastructure; the product library (libbobcat_cuda.so) does not contain it. */
#ifndef BOBCAT_SYNTH_WRITER_H
#define BOBCAT_SYNTH_WRITER_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum { BCS_OK = 0, BCS_ERR_IO = 1, BCS_ERR_ARGUMENT = 13 };
/* ggml type ids of the tensor types the writer can draw. */
enum { BCS_F32 = 0, BCS_Q4_0 = 2, BCS_Q8_0 = 8 };
/* How a tensor's values are drawn: N(0, value^2) from a counter-based generator keyed by (seed,
 * tensor order, row), so the bytes do not depend on thread count; a constant; or
 * -exp(N(0, value^2)) (the stored form of a DeltaNet decay, always negative). */
enum { BCS_INIT_NORMAL = 0, BCS_INIT_CONSTANT = 1, BCS_INIT_NEG_EXP_NORMAL = 2 };

typedef struct bcs_writer bcs_writer;

const char* bcs_last_error(void);
int32_t bcs_writer_new(const char* path, uint64_t seed, bcs_writer** out);
int32_t bcs_writer_kv_u32(bcs_writer* w, const char* key, uint32_t value);
int32_t bcs_writer_kv_f32(bcs_writer* w, const char* key, float value);
int32_t bcs_writer_kv_str(bcs_writer* w, const char* key, const char* value);
int32_t bcs_writer_kv_u32_array(bcs_writer* w, const char* key, const uint32_t* values, uint64_t n);
/* `dims` is innermost-first (ne0 = columns). Quantised types are rounded from the drawn f32 values
 * with ggml's reference rounding. */
int32_t bcs_writer_tensor(bcs_writer* w, const char* name, int32_t type, const uint64_t* dims, uint32_t n_dims, int32_t init,
                          float value);
/* Draws every tensor (in parallel over rows) and writes the file. Frees the writer. */
int32_t bcs_writer_finish(bcs_writer* w);

#ifdef __cplusplus
}
#endif
#endif
