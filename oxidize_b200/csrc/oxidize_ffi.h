/* C ABI of the engine (the surface of the reference's oxidize-ffi crate).
 *
 * The library embeds the Python interpreter the package was built with; the first call starts it (or joins the one that
 * is already running when the library is loaded from Python).  OXIDIZE_PYTHON names another interpreter,
 * OXIDIZE_PACKAGE_ROOT another checkout of the package, OXIDIZE_FFI_DEVICE ("cpu", "cuda:1", ...) the device models load on.  All functions may be called from any thread; calls are
 * serialised by the interpreter lock.
 */
#ifndef OXIDIZE_FFI_H
#define OXIDIZE_FFI_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

const char* oxidize_ffi_version(void);

/* out[rows] = W[rows, cols] * vector[cols]; W packed in the GGML type `quant_type` (0 F32, 1 F16, 2 Q4_0, 8 Q8_0,
 * 12 Q4_K, 14 Q6_K, 30 BF16, ...).  0 on success, negative on a bad argument. */
int32_t oxidize_gemv_quantized(uint32_t quant_type, const uint8_t* qbytes, size_t qbytes_len, size_t rows, size_t cols,
                               const float* vector, float* output);

/* A model from a GGUF file, on the GPU when one is visible; NULL on failure (the reason goes to stderr). */
void* oxidize_model_load(const char* path);
void oxidize_model_free(void* model);
uint32_t oxidize_model_vocab_size(void* model);

/* One sequence: its position and cache. */
void* oxidize_session_new(void);
void oxidize_session_reset(void* session);
void oxidize_session_free(void* session);

/* Feed `n_tokens` tokens at the session's position; the logits that follow the last one are written to
 * logits_out[0 .. vocab).  0 on success; -1 internal error, -2 bad argument, -3 context exhausted. */
int32_t oxidize_model_forward(void* model, void* session, const uint32_t* tokens, size_t n_tokens, float* logits_out,
                              size_t vocab_size);

/* Index of the largest logit (the last one among equals). */
uint32_t oxidize_sample_argmax(const float* logits, size_t vocab_size);

#ifdef __cplusplus
}
#endif
#endif /* OXIDIZE_FFI_H */
