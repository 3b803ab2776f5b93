/*
 * C ABI of libcoli_cuda_backend.so — the B200 (sm_100a) MoE expert-FFN backend.
 *
 * Part 1 declares, with unchanged names and argument lists, every entry point
 * of the reference engine's CUDA backend (cuda/backend_cuda.h:29-192), so that
 * the reference's FFI crate (crates/peregrine-cuda/src/lib.rs:40-145) links
 * against this library without edits.  Part 2 is additive: grouped-int4
 * residency and a device-resident MoE layer (router, permutation, experts and
 * ordered combine with no host round trip).
 *
 * Conventions (cuda/backend_cuda.cu:68-72, 614-619): int results are 1 on
 * success and 0 on failure; nothing throws or aborts; a CUDA failure prints
 * "[CUDA] <what>: <reason>" on stderr; pointer results are NULL on failure;
 * statistic getters accept NULL out-pointers.
 *
 * Numerics of the int4 paths follow the reference's CPU integer-dot kernels
 * (crates/peregrine-kernels/src/{quant,idot,matmul}.rs): activations are
 * quantised to int8 per row, block dots are exact int32, fp32 folding is done
 * in the reference's order without FMA contraction.
 */
#ifndef PEREGRINE_B200_H
#define PEREGRINE_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define COLI_CUDA_MAX_DEVICES 16 /* cuda/backend_cuda.h:21 */

typedef struct ColiCudaTensor ColiCudaTensor; /* cuda/backend_cuda.h:24 */
typedef struct ColiCudaGraph ColiCudaGraph;   /* cuda/backend_cuda.h:27 */

/* =========================================================================
 * Part 1 — the reference surface
 * ========================================================================= */

/* ---- contexts (cuda/backend_cuda.h:30-41; backend_cuda.cu:484-516) ---- */
/* `devices` are CUDA ordinals; duplicates, out-of-range ordinals and count
 * outside 1..16 are rejected.  Re-initialising replaces the context set. */
int coli_cuda_init(const int *devices, int count);
void coli_cuda_shutdown(void);
int coli_cuda_device_count(void);       /* contexts this process initialised */
int coli_cuda_probe_device_count(void); /* devices the driver reports, no init needed */
int coli_cuda_device_at(int index);     /* ordinal of context `index`, -1 if none */
int coli_cuda_mem_info(int device, size_t *free_bytes, size_t *total_bytes);
void coli_cuda_stats(int device, size_t *tensor_count, size_t *tensor_bytes); /* device < 0: all */
void coli_cuda_group_stats(uint64_t *calls, uint64_t *experts, uint64_t *rows, double *h2d_ms, double *kernel_ms,
                           double *d2h_ms); /* times only with COLI_CUDA_PROFILE=1 */

/* ---- residency (cuda/backend_cuda.h:43-52, 132-138; backend_cuda.cu:747-811) ----
 * fmt: 0 = f32 [O,I]; 1 = int8 [O,I] + scales[O]; 2 = int4, two per byte, stored v+8,
 * even element in the low nibble + scales[O]; 3 = int2, four per byte, stored v+2 + scales[O].
 * A call with *tensor already set uploads nothing and reports whether
 * (fmt, I, O, device) match.  The caller's buffers may be freed on return. */
int coli_cuda_tensor_upload(ColiCudaTensor **tensor, const void *weights, const float *scales, int fmt, int I, int O,
                            int device);
int coli_cuda_tensor_update(ColiCudaTensor *tensor, const void *weights, const float *scales);
void coli_cuda_tensor_free(ColiCudaTensor *tensor); /* NULL-safe */
size_t coli_cuda_tensor_bytes(const ColiCudaTensor *tensor);
int coli_cuda_tensor_device(const ColiCudaTensor *tensor);

/* ---- single matrices (cuda/backend_cuda.h:54-71) ---- */
/* y[S,O] = x[S,I] W^T with host x/y; uploads W on first use. */
int coli_cuda_matmul(ColiCudaTensor **tensor, float *y, const float *x, const void *weights, const float *scales,
                     int fmt, int S, int I, int O, int device);
/* y = down(silu(gate x) * up x) for S host rows through three resident tensors. */
int coli_cuda_expert_mlp(ColiCudaTensor *gate, ColiCudaTensor *up, ColiCudaTensor *down, float *y, const float *x,
                         int S);
int coli_cuda_shared_mlp_w4a16(ColiCudaTensor *gate, ColiCudaTensor *up, ColiCudaTensor *down, float *y,
                               const float *x, int S);

/* ---- the expert group: the GPU lane's hot call (cuda/backend_cuda.h:73-110;
 * backend_cuda.cu:1035-1259).  Expert c processes rows[c] >= 1 consecutive
 * host rows of x; y receives sum(rows) rows of width D in the same order.
 * 1 <= count <= 256; all tensors on one device with gate/up [I,D], down [D,I].
 * int4 experts (fmt 2, or grouped via Part 2) run the W4A8 integer path;
 * f32 experts run an fp32 path; the two may be mixed within one call. */
int coli_cuda_expert_group(ColiCudaTensor *const *gates, ColiCudaTensor *const *ups, ColiCudaTensor *const *downs,
                           const int *rows, int count, float *y, const float *x);
/* Same call with the reference's WMMA tile hint.  This backend has one int4 arm,
 * so the tile is accepted and ignored; *arm_out (may be NULL) reports the
 * reference's arm code a caller would expect for the call: 1 when
 * COLI_CUDA_TC_W4A16 is set and every expert is int4 with rows >= the W4A16
 * minimum, else 2 for all-int4 groups and 3 otherwise. */
int coli_cuda_expert_group_tiled(ColiCudaTensor *const *gates, ColiCudaTensor *const *ups,
                                 ColiCudaTensor *const *downs, const int *rows, int count, float *y, const float *x,
                                 int tile_m, int tile_n, int tile_k, int *arm_out);
/* Same call followed by the CSR combine on the device: out[s,:] (s < s_n) is the
 * sum, in listed order and starting from zero, of rw[j] * y[j,:] over
 * j = row_idx[row_ptr[s] .. row_ptr[s+1]).  No atomics: identical bits every run. */
int coli_cuda_expert_group_reduce(ColiCudaTensor *const *gates, ColiCudaTensor *const *ups,
                                  ColiCudaTensor *const *downs, const int *rows, int count, const int *row_ptr,
                                  const int *row_idx, const float *rw, int s_n, float *out, const float *x);

/* ---- attention (cuda/backend_cuda.h:112-130, 161-176).  Outside the expert-FFN
 * path: exported so the reference's FFI links; every one reports failure (0),
 * which the reference's callers treat as "compute this on the CPU lane". ---- */
int coli_cuda_attention_absorb(ColiCudaTensor *kv_b, float *ctx, const float *q, const float *latent,
                               const float *rope, int H, int Q, int R, int V, int K, int T, float attention_scale);
int coli_cuda_attention_absorb_batch(ColiCudaTensor *kv_b, float *ctx, const float *q, const float *latent,
                                     const float *rope, int S, int H, int Q, int R, int V, int K, int T,
                                     float attention_scale);
int coli_cuda_attention_project_batch(ColiCudaTensor *kv_b, ColiCudaTensor *o_proj, float *out, const float *q,
                                      const float *latent, const float *rope, int S, int H, int Q, int R, int V,
                                      int K, int T, float attention_scale);
int coli_cuda_attention_project_batch_dev(ColiCudaTensor *kv_b, ColiCudaTensor *o_proj, float *out,
                                          const float *q_dev, const float *latent_dev, const float *rope_dev, int S,
                                          int H, int Q, int R, int V, int K, int T, float scale);
int coli_cuda_attention_absorb_batch_dev(ColiCudaTensor *kv_b_shard, float *ctx_dev, const float *q_dev,
                                         const float *latent_dev, const float *rope_dev, int S, int H, int Q, int R,
                                         int V, int K, int T, float scale);
int coli_cuda_attention_absorb_kvdev(ColiCudaTensor *kv_b, float *ctx, const float *q, const float *latent_dev,
                                     const float *rope_dev, int H, int Q, int R, int V, int K, int T, float scale);
int coli_cuda_attention_project_batch_dev_out(ColiCudaTensor *kv_b, ColiCudaTensor *o_proj, float *out_dev,
                                              const float *q_dev, const float *latent_dev, const float *rope_dev,
                                              int S, int H, int Q, int R, int V, int K, int T, float scale);

/* ---- device-pointer primitives on the context's stream (cuda/backend_cuda.h:140-177) ---- */
float *coli_cuda_pipe_scratch(int device, int slot, size_t bytes); /* 24 grow-only slots */
void *coli_cuda_pipe_alloc(int device, size_t bytes);
void coli_cuda_pipe_free(int device, void *p);
int coli_cuda_pipe_upload(int device, void *dst, const void *src, size_t bytes);
int coli_cuda_pipe_download(int device, const void *src, void *dst, size_t bytes);
int coli_cuda_pipe_rmsnorm(int device, float *y_dev, const float *x_dev, const float *w_dev, int S, int D, float eps);
int coli_cuda_pipe_rmsnorm_s(int device, float *y_dev, const float *x_dev, const float *w_dev, int S, int D,
                             float eps, int xstride, int ystride);
int coli_cuda_pipe_rope(int device, float *v_dev, const int *pos_dev, int rows, int stride, int offset, int R,
                        int heads, float theta);
int coli_cuda_pipe_rope_base(int device, float *v_dev, int pos_base, int rows, int stride, int offset, int R,
                             int heads, float theta);
int coli_cuda_pipe_silu_mul(int device, float *gate_dev, const float *up_dev, size_t n);
int coli_cuda_pipe_add(int device, float *x_dev, const float *t_dev, size_t n);
int coli_cuda_pipe_rows_add(int device, float *x_dev, const float *partial_dev, const int *rows_dev, int nrows,
                            int D);
int coli_cuda_pipe_gemm(ColiCudaTensor *t, float *y_dev, const float *x_dev, int S);
int coli_cuda_pipe_copy2d(int device, float *dst, int dpitch, const float *src, int spitch, int width, int height);
int coli_cuda_pipe_peer_copy(int dst_dev, float *dst, int src_dev, const float *src, size_t bytes);
int coli_cuda_pipe_sync(int device);

/* ---- stream capture (cuda/backend_cuda.h:179-191) ---- */
int coli_cuda_graph_begin(int device);
int coli_cuda_graph_end(int device, ColiCudaGraph **out);
int coli_cuda_graph_launch(ColiCudaGraph *g);
void coli_cuda_graph_free(ColiCudaGraph *g);
/* Counters of the expert-group graph cache (COLI_CUDA_GRAPH=1). */
void coli_cuda_graph_cache_stats(uint64_t *captures, uint64_t *replays, uint64_t *invalidations,
                                 uint64_t *uncacheable);

/* =========================================================================
 * Part 2 — additive entry points (no counterpart in cuda/backend_cuda.h)
 * ========================================================================= */

/* Grouped int4 residency.  The reference keeps this format on the CPU only
 * (crates/peregrine-core/src/qt.rs:70-85; crates/peregrine-kernels/src/idot.rs:78-110)
 * and dequantises it to f32 before upload (crates/peregrine-model/src/gpu.rs:1373-1382).
 * weights: [O, ceil(I/2)] as fmt 2; scales: [O * ceil(I/gs)], row o group g at
 * o*ng+g; gs a multiple of 32, at most 256.  The handle works everywhere a
 * fmt-2 handle does and reports fmt 4. */
int coli_cuda_tensor_upload_grouped(ColiCudaTensor **tensor, const void *weights, const float *scales, int I, int O,
                                    int gs, int device);

/* One resident MoE layer: router + E routed experts (+ one shared expert).
 * Mirrors the arguments of the reference's layer forward
 * (crates/peregrine-model/src/mlp.rs:46-57, MoeCfg :33-39;
 * crates/peregrine-model/src/concurrent.rs:1200). */
typedef struct ColiCudaMoeLayer ColiCudaMoeLayer;

/* router_w: host fp32 [E, D]; router_bias: host fp32 [E] (NULL = zeros). */
int coli_cuda_moe_layer_create(ColiCudaMoeLayer **layer, int device, int D, int I, int E, int k, int norm_topk,
                               float routed_scale, const float *router_w, const float *router_bias);
/* Attach expert `e` (0..E-1 routed, E = the shared expert).  The layer borrows the
 * tensors; they must outlive it.  All experts must be int4 (fmt 2 or grouped) of
 * one format, gate/up [I, D], down [D, I]. */
int coli_cuda_moe_layer_set_expert(ColiCudaMoeLayer *layer, int e, ColiCudaTensor *gate, ColiCudaTensor *up,
                                   ColiCudaTensor *down);
void coli_cuda_moe_layer_free(ColiCudaMoeLayer *layer);

/* out[M, D] = MoE(x[M, D]) with device pointers (row strides D), enqueued on the
 * device's stream with no host synchronisation: route -> batch union -> pair
 * layout -> quantise -> gate/up + SwiGLU -> quantise -> down -> ordered combine.
 * Workspace grows (allocates) on the first call at a larger M. */
int coli_cuda_moe_layer_forward_dev(ColiCudaMoeLayer *layer, float *out_dev, const float *x_dev, int M);
/* Same with host pointers: copies x in, runs, copies out, blocks until done. */
int coli_cuda_moe_layer_forward(ColiCudaMoeLayer *layer, float *out, const float *x, int M);

/* Inspection of the last forward (blocking copies to host; any pointer may be NULL).
 * idx, w: [M*k]; keff: [M]; union_ids: [E] with *n_union entries. */
int coli_cuda_moe_layer_last_routing(ColiCudaMoeLayer *layer, int M, int *idx, float *w, int *keff, int *union_ids,
                                     int *n_union);
/* When enabled, the next forwards also record the per-block int32 accumulators of
 * every (pair, output, group).  Sizes for M tokens: gate/up taps
 * [pairs][2][I][ng(D)] and down taps [pairs][D][ng(I)], pairs as reported by
 * coli_cuda_moe_layer_last_pairs.  For per-row (fmt 2) experts ng is 1 and the tap
 * is the whole-row accumulator. */
int coli_cuda_moe_layer_enable_taps(ColiCudaMoeLayer *layer, int enable);
/* Speculative routing of decode-sized batches (at most 2 tokens, one device): the expert launches
 * start from a selection made on parallel-sum logits while the exact sequential router chains
 * (crates/peregrine-kernels/src/matmul.rs:18-30) run beside them; weights, combine order and the
 * selection check come from the exact chains, and a disagreement is recomputed, so results do not
 * depend on the mode.  mode: -1 process default (on unless PEREGRINE_B200_SPEC_ROUTE=0), 0 off,
 * 1 on, 2 on with the speculative pick deliberately wrong (exercises the recompute path). */
int coli_cuda_moe_layer_set_spec(ColiCudaMoeLayer *layer, int mode);
/* A single token on one device with speculative routing on takes the whole step — routing, gate/up,
 * down, ordered combine — in ONE launch of one CTA per SM (no counterpart in the reference, whose
 * step is a host loop over kernels, cuda/backend_cuda.cu:1035-1211).  mode: -1 process default (on
 * unless PEREGRINE_B200_FUSED_DECODE=0), 0 separate launches, 1 one launch.  Results are identical
 * either way; taps and per-launch profiling always use the separate launches. */
int coli_cuda_moe_layer_set_fused(ColiCudaMoeLayer *layer, int mode);
/* Inspection of the single-launch step: with `enable` set, the next such step records 16 device
 * timer stamps (ns) per CTA; a later call with `stamps` (capacity_ctas * 16 values) reads them back.
 * n_ctas / n_chain report the launch's CTA count and how many of them run the exact router. */
int coli_cuda_moe_layer_decode_timeline(ColiCudaMoeLayer *layer, int enable, unsigned long long *stamps,
                                        int capacity_ctas, int *n_ctas, int *n_chain);
/* pair_token[p] = token of pair row p, pair_expert[p] = expert id (E = shared). */
int coli_cuda_moe_layer_last_pairs(ColiCudaMoeLayer *layer, int *n_pairs, int *pair_token, int *pair_expert,
                                   int capacity);
int coli_cuda_moe_layer_read_taps(ColiCudaMoeLayer *layer, int32_t *gateup_taps, size_t gateup_count,
                                  int32_t *down_taps, size_t down_count);

/* Measurement aids (no counterpart in the reference).  int8_peak_probe: tera-ops per second of a
 * bare tcgen05.mma kind::i8 loop, one CTA per SM (the measured denominator of the prefill roofline).
 * set_bias: replaces a resident layer's selection bias (host fp32 [E]). */
double coli_cuda_int8_peak_probe(int device, int iters, int launches);
/* A second resident copy of a tensor made on the device (*out must be NULL): synthetic stacks fill
 * their layers with distinct memory without repacking every expert on the host. */
int coli_cuda_tensor_clone(ColiCudaTensor **out, const ColiCudaTensor *src);
int coli_cuda_moe_layer_set_bias(ColiCudaMoeLayer *layer, const float *router_bias);

/* Two device-pointer primitives the decode loop around the FFN needs, in the style of the pipe_* family
 * (no counterpart in cuda/backend_cuda.h; the reference does both on the host):
 * embedding row gather x_dev[s,:] = table_dev[ids_dev[s],:] (fp32 table [V, D]) and greedy
 * pick ids_dev[s] = argmax(logits_dev[s,:V]) with the rules of crates/peregrine-model/src/sample.rs:21-32
 * (first non-NaN start, strict '>', lowest index wins, all-NaN row -> 0). */
int coli_cuda_pipe_embed(int device, float *x_dev, const float *table_dev, const int *ids_dev, int S, int D, int V);
int coli_cuda_pipe_argmax(int device, int *ids_dev, const float *logits_dev, int S, int V);

/* Expert parallelism over the GPUs of one node (the reference has none: crates/peregrine-model/src/gpu.rs:1454-1457
 * hard-codes one device; docs/scale-out-design.md:34-72 sketches an owner map per (layer, expert) and requires
 * cross-device partial sums in fixed order).  Rank r of `world` owns the routed experts
 * [r*ceil(E/world), (r+1)*ceil(E/world)) and only those need to be attached; router and shared expert are
 * replicated; the batch of M tokens is data-parallel, rank r holding tokens [r*M/world, (r+1)*M/world).
 * A layer step is four phases on the rank's stream, exchanging through blocks of peer-visible memory:
 * route the home tokens and publish their picks; plan the batch and send each (token, expert) pair's
 * int8 row to the expert's owner; compute the owned experts and return the un-weighted rows to the
 * tokens' home ranks; combine the home tokens in batch-union order, shared expert last.  Every
 * transfer is a store into the peer's block followed by a flag; every wait is bounded and reports
 * through coli_cuda_last_device_error. */
typedef struct ColiCudaEp ColiCudaEp;
int coli_cuda_moe_layer_set_ep(ColiCudaMoeLayer *layer, int rank, int world);
/* The exchange block of one rank for batches of M tokens (M a multiple of world) of width D, top-k. */
int coli_cuda_ep_create(ColiCudaEp **ep, int device, int rank, int world, int M, int D, int k);
size_t coli_cuda_ep_block_bytes(const ColiCudaEp *ep);
void *coli_cuda_ep_local_base(const ColiCudaEp *ep);
/* One process per GPU: export a 64-byte handle, hand it to the other ranks, attach theirs. */
int coli_cuda_ep_export(ColiCudaEp *ep, void *handle64);
int coli_cuda_ep_attach(ColiCudaEp *ep, int peer_rank, const void *handle64);
/* Blocks the process can already address (ranks emulated on one device; devices of one process). */
int coli_cuda_ep_attach_ptr(ColiCudaEp *ep, int peer_rank, void *base);
void coli_cuda_ep_free(ColiCudaEp *ep);
/* The ranks must enter a step within the device-side wait limit (about a second) of each other: after
 * set-up of uneven length they meet once on the host before the first step.  A wait that runs out
 * sets the device error word and makes every later wait of that rank give up at once; when all ranks
 * have drained and met again, each calls this to clear that state. */
int coli_cuda_ep_reset(ColiCudaEp *ep);
int coli_cuda_moe_layer_ep_route_dev(ColiCudaMoeLayer *layer, ColiCudaEp *ep, const float *x_loc_dev);
int coli_cuda_moe_layer_ep_dispatch_dev(ColiCudaMoeLayer *layer, ColiCudaEp *ep);
int coli_cuda_moe_layer_ep_experts_dev(ColiCudaMoeLayer *layer, ColiCudaEp *ep);
int coli_cuda_moe_layer_ep_finish_dev(ColiCudaMoeLayer *layer, ColiCudaEp *ep, float *out_loc_dev);
/* All four phases: out_loc_dev[M/world, D] = layer(x_loc_dev[M/world, D]) for this rank's home tokens. */
int coli_cuda_moe_layer_ep_forward_dev(ColiCudaMoeLayer *layer, ColiCudaEp *ep, float *out_loc_dev,
                                       const float *x_loc_dev);

/* Profile mode (in the spirit of COLI_CUDA_PROFILE, cuda/backend_cuda.cu:1068,1174-1207):
 * each forward brackets its seven launches with events, waits for the stream and
 * accumulates per-stage device milliseconds: quantise x, router logits, routing plan,
 * gate/up GEMV, quantise h, down GEMV, combine.  Switching resets the accumulators. */
/* Host-side microseconds of coli_cuda_moe_layer_forward since the last reset, by part: staging copy of
 * x, enqueueing the upload, enqueueing the launches, waiting for the device, copying the result out. */
int coli_cuda_moe_layer_host_times(ColiCudaMoeLayer *layer, double *us5, uint64_t *calls, int reset);
/* coli_cuda_graph_launch (which waits for the stream, as the reference's does) without the wait. */
int coli_cuda_graph_launch_async(ColiCudaGraph *g);

int coli_cuda_moe_layer_set_profile(ColiCudaMoeLayer *layer, int enable);
int coli_cuda_moe_layer_profile(ColiCudaMoeLayer *layer, double *stage_ms7, uint64_t *calls);

/* The int4 product of coli_cuda_pipe_gemm for callers that must not allocate.  It has no
 * counterpart in the reference (cuda/backend_cuda.h has no allocation-free entry).  Same
 * arguments and result as coli_cuda_pipe_gemm for an int4 tensor (fmt 2 or grouped): y_dev[S,O] =
 * x_dev[S,I] W^T, device pointers, enqueued on the device's stream.  Its scratch (int8 copy of
 * x, row scales, block sums, slot table) is a 1 MiB array inside the library image instead
 * of cudaMalloc'ed buffers, so it calls no cudaMalloc/cudaFree: meant for a decode lane that
 * runs with VRAM fully committed to experts, or where a device-wide synchronising call is
 * not allowed.  Requests whose scratch exceeds 1 MiB (about S*I*1.2 bytes; S <= 143 at
 * I = 6144) are refused with a message.  The first call on a device resolves the array's
 * address and configures the kernels; all calls on a device share the array, so calls that
 * overlap on the GPU race. */
int coli_cuda_pipe_gemm_noalloc(ColiCudaTensor *t, float *y_dev, const float *x_dev, int S);

/* Device error word of a context: 0 when no kernel reported a problem since the
 * last call; otherwise the code (1 = a bounded wait on a copy barrier expired). */
int coli_cuda_last_device_error(int device);
/* Self-test of the failure path every kernel of this library shares: launches one CTA that waits,
 * with a limit of `limit_cycles` clock cycles, on a copy barrier that nothing will ever complete;
 * the wait gives up, the kernel reports code 1 through the device error word and returns, and the
 * context stays usable.  Returns 1 when the launch and its synchronise succeeded (the caller then
 * reads coli_cuda_last_device_error).  No counterpart in the reference. */
int coli_cuda_selftest_bounded_wait(int device, long long limit_cycles);
/* Number of this library's kernels launched since init (all devices). */
uint64_t coli_cuda_kernel_launches(void);
/* The context's stream as a cudaStream_t, for callers that order their own work. */
void *coli_cuda_stream(int device);

#ifdef __cplusplus
}
#endif
#endif /* PEREGRINE_B200_H */
