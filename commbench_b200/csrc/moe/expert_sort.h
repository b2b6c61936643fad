// Stable sort of MoE (token, k) selections by expert id.
//
// Given topk_idx[n_pairs] (expert id per selection, negative = masked) the result is
//   counts[E]            selections per expert
//   sorted_pair[n_pairs] selection indices grouped by expert (ascending expert id), in
//                        their original order inside each group; masked selections are
//                        not listed, the tail of the array is left untouched.
// The order is a pure function of the input (no atomics decide positions), which is what
// the deterministic dispatch needs.  Scratch: one int per selection plus one per expert.
#pragma once

#ifdef __cplusplus
extern "C" {
#endif

// Scratch supplied by the caller: `scratch` holds at least (n_pairs + E) ints of device
// memory.  Returns 0, or -1 with the reason in cb_last_error().
int cb_moe_expert_sort(const void* topk_idx, int n_pairs, int E, void* scratch, void* sorted_pair,
                       void* counts, void* stream);

// Largest problem the variant below accepts.
#define CB_EXPERT_SORT_STATIC_MAX_PAIRS 262144
#define CB_EXPERT_SORT_STATIC_MAX_EXPERTS 1024

#ifdef __cplusplus
}
#endif
