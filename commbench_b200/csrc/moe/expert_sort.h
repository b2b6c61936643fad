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

// Same result as cb_moe_expert_sort, for callers that must not allocate.  (This entry
// point has no counterpart in the reference.)
//
// Who needs it: a serving loop that has handed every spare byte of HBM to its KV cache and
// treats any allocation after warm-up as a bug; a plug-in living inside another framework's
// memory pool, where a cudaMalloc of its own would synchronise the whole device or simply
// fail; code on a latency-critical stream that cannot afford the implicit synchronisation
// an allocation brings.  Such callers pass inputs and outputs only.
//
// The scratch ((MAX_PAIRS + MAX_EXPERTS) ints, about 1.05 MB) is a file-scope device array
// inside the library: every GPU that loads the library holds it until the process exits.
// The function calls no cudaMalloc / cudaFree and no allocating library routine.
//
//  * n_pairs <= CB_EXPERT_SORT_STATIC_MAX_PAIRS and E <= CB_EXPERT_SORT_STATIC_MAX_EXPERTS,
//    otherwise -1 and an error text.
//  * The first call on each device looks up the array's device address (one
//    cudaGetSymbolAddress with that device current); make that first call before any
//    stream capture begins.
//  * All calls on a device share the one array and it keeps the previous call's contents.
//    Nothing in it has to start at zero (every word that is read was written earlier in the
//    same call), but two calls whose kernels overlap on the GPU (different streams) race:
//    serialise them.
int cb_moe_expert_sort_noalloc(const void* topk_idx, int n_pairs, int E, void* sorted_pair,
                               void* counts, void* stream);

#ifdef __cplusplus
}
#endif
