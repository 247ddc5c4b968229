/* C API of the engine: create an instance, generate, free.
 *
 * Counterpart of the reference's `libxllm.so` C interface (xllm/c_api/llm.h, types.h) and of its
 * C++ wrapper (xllm/cc_api/llm.h): a host program that is not written in Python links this library
 * and drives the engine in-process.  The engine itself is the Python package `xllm_b200`; the
 * library embeds (or joins) a CPython interpreter and forwards every call to
 * `xllm_b200.api.c_bridge`.  Strings are UTF-8; results are JSON documents owned by the caller
 * until passed to xllm_free_string().
 */
#ifndef XLLM_B200_C_API_H_
#define XLLM_B200_C_API_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define XLLM_C_API __attribute__((visibility("default")))
#else
#define XLLM_C_API
#endif

typedef struct xllm_llm xllm_llm;

/* options_json: keyword arguments of xllm_b200.LLM as a JSON object, e.g.
 *   {"devices": "cuda:0", "dtype": "bfloat16", "block_size": 16, "max_seqs_per_batch": 256}
 * Returns NULL on failure; xllm_last_error() then tells why. */
XLLM_C_API xllm_llm* xllm_llm_create(const char* model, const char* options_json);
XLLM_C_API void xllm_llm_destroy(xllm_llm* llm);

/* prompts_json: a JSON array whose elements are strings or arrays of token ids.
 * sampling_json: fields of SamplingParams, e.g. {"max_tokens": 64, "temperature": 0.0}.
 * Returns a JSON array with one object per prompt:
 *   {"token_ids": [...], "text": "...", "finish_reason": "...", "prompt_tokens": n}  */
XLLM_C_API char* xllm_llm_generate(xllm_llm* llm, const char* prompts_json, const char* sampling_json);

/* Every other method of the offline API by name; args_json holds its keyword arguments, the result is
 * a JSON document:
 *   "chat"           {"messages": [{"role": ..., "content": ...}, ...], "sampling": {...}}  -> same objects as generate
 *   "embed"          {"prompts": [...]}                                -> [[float, ...], ...]
 *   "beam_search"    {"prompt": [...ids] | "text", "beam_width": 4, "max_tokens": 16} -> [{"token_ids", "score"}, ...]
 *   "sleep"          {"level": 1 | 2}     "wake_up" {}     "stats" {}   -> {"ok": true} / counters  */
XLLM_C_API char* xllm_llm_call(xllm_llm* llm, const char* method, const char* args_json);

/* Engine counters as a JSON object (steps, KV utilisation, prefix hits, ...). */
XLLM_C_API char* xllm_llm_stats(xllm_llm* llm);

XLLM_C_API void xllm_free_string(char* s);
XLLM_C_API const char* xllm_last_error(void);

#ifdef __cplusplus
}
#endif
#endif
