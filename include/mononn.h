/* C ABI of libmononn_b200.so: the B200 (sm_100a) backend for the MonoNN hot path
 * "XLA HLO module in -> one persistent kernel -> one launch per inference".
 *
 * Conventions
 *   - every function returns 0 on success and a negative MONONN_ERR_* code on failure;
 *     nothing here aborts the process (the reference LOG(FATAL)s instead) and there is
 *     no CPU fallback: without a usable sm_100 device the calls fail.
 *   - pointers are borrowed for the duration of the call unless the parameter is `out`.
 *   - different modules may be used from different threads; one module from one
 *     thread at a time. Launches of one module must be ordered on the GPU (one stream, or
 *     streams chained by events): a module owns one barrier counter and one stage table.
 *   - every call runs on the module's device and restores the caller's current device.
 */
#ifndef MONONN_B200_H_
#define MONONN_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum {
  MONONN_OK = 0,
  MONONN_ERR_INVALID_ARGUMENT = -1,
  MONONN_ERR_PARSE = -2,           /* HLO text or spec JSON is malformed */
  MONONN_ERR_UNSUPPORTED = -3,     /* op / dtype / layout / pattern outside the supported set */
  MONONN_ERR_CUDA = -4,            /* a CUDA runtime or driver call failed */
  MONONN_ERR_NO_DEVICE = -5,       /* no sm_100 device */
  MONONN_ERR_BARRIER_TIMEOUT = -6, /* a bounded wait inside the kernel expired */
  MONONN_ERR_CONSTANT = -7,        /* unknown constant name or wrong size */
  MONONN_ERR_IO = -8,              /* spec / dump directory I/O */
  MONONN_ERR_NOT_READY = -9,       /* launch before all constants were set */
  MONONN_ERR_TOO_LARGE = -10       /* size beyond a documented maximum */
};

typedef struct mononn_module mononn_module; /* opaque; free with mononn_destroy */

/* Replaces the environment + Config singleton of the reference
 * (mononn_engine/config/config.h:19-53, EnvVars.md:4-16). NULL strings fall back to the
 * environment variables TF_MONONN_DUMP_DIR / TF_MONONN_EXISTING_TUNING_SPEC_DIR /
 * TF_MONONN_THREADPOOL_SIZE. */
typedef struct {
  int device;                   /* CUDA device ordinal (the reference hard-codes 0) */
  const char* dump_dir;         /* where tune() writes specs and reports */
  const char* spec_dir;         /* existing tuning spec to load instead of tuning */
  int threadpool_size;          /* host threads that re-pack weights into tiles whenever a plan is
                                   (re)loaded, i.e. per tuning candidate; 0 = all cores */
  int tuning_level;             /* what mononn_tune searches: 0 nothing (times the heuristic spec),
                                   1 stage structure (qkv_fusion, row_fusion) and per-GEMM-class
                                   tiles timed on their own stage, 2 + the number of CTAs */
  unsigned barrier_timeout_us;  /* bound on every in-kernel wait; 0 = 2 000 000 */
} mononn_options;

typedef struct {
  int index;        /* position in the kernel argument list */
  size_t bytes;
  int kind;         /* 0 parameter, 1 live-out, 2 temp */
  int param_number; /* HLO parameter_number for kind 0, live-out ordinal for kind 1 */
} mononn_arg_desc;

/* Parse -> fuse -> (load spec | heuristics) -> stage table.
 * Replaces IRParserFused::from_hlo_module_unique + OptimizationRunner::run_group_* +
 * GraphCodegen::generate as driven by MonoNNModule::generate_code
 * (mononn_engine/module/mononn_module.cc:39-159) and the spec-loading side of the
 * TF_MONONN_EXISTING_TUNING_SPEC_DIR hook (README.md:145-149). */
int mononn_compile_hlo_text(const char* hlo_text, size_t len, const char* kernel_name,
                            const mononn_options* options, mononn_module** out);

/* Standalone path: build the fused graph of an encoder family from a JSON configuration
 * instead of an HLO dump, e.g. {"model":"bert","layers":12,"hidden":768,"heads":12,
 * "ffn":3072,"vocab":30522,"max_pos":512,"types":2,"batch":1,"seq":128,"eps":1e-12,
 * "act":"gelu_erf"}. The model definitions are those the reference exports in
 * examples/utils/save_model.py:44-110; constants are named "embeddings.word",
 * "layer<i>.attn.q.w", ... (mononn_constant_info lists them). */
int mononn_compile_encoder_json(const char* config_json, const char* kernel_name,
                                const mononn_options* options, mononn_module** out);

/* Kernel argument list: parameters by parameter_number, live-outs, then temp
 * (mononn_engine/module/mononn_module.cc:91-143, README.md:186-200). */
int mononn_module_args(const mononn_module* m, const mononn_arg_desc** descs, int* n);

/* grid_dim, block_dim, dynamic shared memory: GraphSpecification.cuda_context.
 * cuda_runtime_context (mononn_engine/core/context/cuda_runtime_context.cc:32-55). */
int mononn_module_launch_config(const mononn_module* m, unsigned grid[3], unsigned block[3],
                                unsigned* smem_bytes);

/* Non-scalar HLO constants (the frozen weights). Replaces the
 * `__device__ uint8_t buffer_for_<name>[bytes]` module globals the TF side fills
 * (mononn_engine/codegen/graph_codegen.cc:71-86). `host` is row-major in the HLO shape. */
int mononn_set_constant(mononn_module* m, const char* hlo_constant_name, const void* host,
                        size_t bytes);
/* Number of constants and the i-th constant's name / byte size. */
int mononn_constant_count(const mononn_module* m, int* n);
int mononn_constant_info(const mononn_module* m, int i, const char** name, size_t* bytes);

/* Exactly one kernel launch on `cuda_stream` (a cudaStream_t), asynchronous.
 * Mirrors the launch sequence of mononn_engine/module/mononn_module_tuner.cc:99-150.
 * device_args[i] follows mononn_module_args order. The first launch with a new set of
 * argument pointers also uploads the re-bound stage table on the same stream. */
int mononn_launch(mononn_module* m, void* const* device_args, int n, void* cuda_stream);

/* One inference from and to HOST memory, the shape of the reference's user-facing call
 * (`sess.run` on host tensors, examples/run_mononn.py:72-84): copies host_inputs[k] (one per
 * parameter, by parameter number) into device_args, launches once, copies every live-out
 * into host_outputs[j], reads the kernel's status word and waits for `cuda_stream`. Pinned
 * host buffers make the copies asynchronous. Where device_args[i] IS the host buffer (pinned
 * memory is device-addressable under unified addressing) no copy is issued: the kernel reads
 * the parameter from, or writes the live-out to, host memory directly. Returns MONONN_ERR_BARRIER_TIMEOUT (and restores
 * the module) when a bounded wait expired in the kernel. */
int mononn_infer_host(mononn_module* m, const void* const* host_inputs, int n_inputs,
                      void* const* host_outputs, int n_outputs, void* const* device_args, int n,
                      void* cuda_stream);

/* Synchronises the device, then reports the kernel's status word: 0, or
 * MONONN_ERR_BARRIER_TIMEOUT with the stage and CTA that gave up. */
int mononn_last_status(mononn_module* m, int* stage, int* cta);

/* Search tile shapes on the device (MonoNNModuleTuner::tune,
 * mononn_engine/module/mononn_module_tuner.cc:620-991): per-GEMM candidates timed in
 * isolation with the allow-list mechanism, best ones merged, end-to-end pick. Needs all
 * constants set and a full argument list. Writes dump_dir/<cluster>/ when set. */
int mononn_tune(mononn_module* m, void* const* device_args, int n, void* cuda_stream);

/* Writes <dir>/<cluster_N>/best_tuning_spec.json (+ performance_report.csv when known):
 * the layout of mononn_engine/module/mononn_module_tuner.cc:584-603. */
int mononn_save_spec(const mononn_module* m, const char* dir);
/* JSON of the current spec; the pointer stays valid until the next call on `m`. */
int mononn_spec_json(mononn_module* m, const char** json);

/* Per-stage device time of the last profiled launch (performance_report.csv,
 * mononn_engine/module/mononn_module_tuner.cc:422-448): launches once with in-kernel
 * %globaltimer stamps, synchronises, fills up to `cap` entries of microseconds and sets
 * *n_stages. names[i] points into module storage. */
int mononn_profile_stages(mononn_module* m, void* const* device_args, int n, void* cuda_stream,
                          double* us, const char** names, int cap, int* n_stages);

/* Inspection. mononn_plan_json: the lowered stage table (stages, operators with tiles,
 * tensor placements, constant bindings) of a module; stands in for the `<context>_src/`
 * dump of the reference (mononn_engine/module/mononn_module_tuner.cc:560-575), since the
 * table is the artefact. mononn_describe lowers without touching a device (kind "hlo" or
 * "encoder", optional spec JSON, SM count) and returns {"plan":..,"spec":..} in a string
 * the caller frees with mononn_free_string. */
int mononn_plan_json(mononn_module* m, const char** json);
int mononn_describe(const char* kind, const char* text, size_t len, const char* spec_json,
                    unsigned sm_count, char** out_json);
void mononn_free_string(char* s);

/* Runs only stages [stage_begin, stage_end) in one launch: the single-node isolation of
 * the reference's codegen_allow_list (mononn_engine/tuning/tuning_space_generator.cc:405-414)
 * used for per-stage timing and for checking intermediate tensors. */
int mononn_launch_stages(mononn_module* m, void* const* device_args, int n, void* cuda_stream,
                         unsigned stage_begin, unsigned stage_end);

/* Per-CTA event trace of one launch: out[(cta * n_stages + stage) * 16 + event] in
 * nanoseconds since the earliest event (0 = event did not occur). Events: 0 epilogue warps
 * passed the previous barrier, 1 finished the stage's items, 2 arrived at the barrier,
 * 3 activation producer passed the barrier, 4 issued its last activation load, 5 MMA issuer
 * saw its first operands, 6 committed its last MMA, 7 weight producer issued its last load,
 * 8..15 finer marks inside the epilogue / row-wise code.
 * This is how the barrier's share of kernel time is measured without a profiler
 * (the reference's performance_report.csv isolates nodes instead,
 * mononn_engine/module/mononn_module_tuner.cc:422-448). cap counts doubles. */
int mononn_trace_stages(mononn_module* m, void* const* device_args, int n, void* cuda_stream,
                        double* out, size_t cap, int* grid, int* n_stages);

/* Test aid (host-side fault injection, no GPU fault involved): the next launch waits for
 * `missing_arrivals` grid-barrier arrivals that no CTA will make, so its first bounded wait
 * expires after barrier_timeout_us; the kernel then drains, returns, and
 * mononn_last_status reports MONONN_ERR_BARRIER_TIMEOUT and restores the module. */
int mononn_debug_skew_barrier(mononn_module* m, unsigned missing_arrivals);

/* Measurement aid: cycles per tcgen05.mma (128 x n x 16, f16 in, f32 accumulate) issued from
 * operands resident in shared memory, on `ctas` CTAs (one per SM) at once: `count` instructions
 * cycling through `accumulators` TMEM buffers, one commit at the end. mode bits (each mode is a
 * separately compiled kernel, so that no run-time test sits in the timed loop):
 *   0  a commit after every four instructions
 *   1  a satisfied mbarrier wait + tcgen05 fence before every four (bits 0 and 1 together are the
 *      bookkeeping of the kernel's main loop)
 *   2  M = 64 instead of 128
 *   3  the A operand is read from tensor memory instead of shared memory
 *   4  the instruction is written without the optional disable-output-lane vector
 *   5  the whole warp runs the loop converged and one elected lane issues (otherwise one lane
 *      runs it alone, diverged from the other 31)
 *   6  the operand descriptors are rebuilt for every group of four from a ring-slot index
 * cycles_per_mma covers first issue .. commit observed, issue_cycles_per_mma the issuing
 * thread alone. The issue loop of the kernel's MMA role and the GEMM tile menu of the tuner are
 * designed from this table; the reference times whole CUTLASS tiles instead
 * (mononn_engine/core/op_impl/gemm_impl.cc:505-566). */
int mononn_debug_mma_issue(int device, unsigned n, unsigned count, unsigned accumulators,
                           unsigned mode, unsigned ctas, double* cycles_per_mma,
                           double* issue_cycles_per_mma, double* ns_per_mma);

/* Algorithmic bytes and FLOPs of one inference (weights once + gathered rows + I/O). */
int mononn_module_cost(const mononn_module* m, double* bytes, double* flops);

/* Allocation-free attention (no counterpart in the reference, which leaves every buffer to
 * XLA's allocator and never allocates on its own).
 *
 * For hosts where this library must not call cudaMalloc: under TensorFlow/XLA the framework's
 * allocator normally owns the whole GPU, so an allocation made by a plug-in can fail or
 * fragment the pool, and serving threads avoid cudaMalloc because it synchronises the device.
 * The call runs one attention stage of the persistent kernel,
 *     out[b, s, h*64:(h+1)*64] = softmax(scale * Q_h K_h^T + (1 - mask) * mask_scale) V_h,
 * on caller-owned f16 buffers and keeps everything else the kernel needs (stage table, tensor
 * maps, barrier counter, status word, the f32 additive mask) in a static device array of
 * 2 KB + 4 * MONONN_NOALLOC_MAX_TOKENS bytes that every GPU loading the library holds until exit.
 *   q, k   f16 [batches*seq, ld_qk], head h in columns h*64 .. h*64+63
 *   v_t    f16 [batches*heads*64, ld_vt]: V transposed per batch (row = b*heads*64 + h*64 + d,
 *          column = key position)
 *   mask   int32 [batches, seq] or NULL;  out  f16 [batches*seq, ld_out]
 * Limits: seq <= 128, head dimension 64, batches*seq <= MONONN_NOALLOC_MAX_TOKENS (larger
 * sizes return MONONN_ERR_TOO_LARGE); base addresses and row pitches multiples of 16 bytes.
 * The call is asynchronous on `cuda_stream` and allocates nothing. All calls on a device
 * share the static array and rewrite it: calls that overlap on the GPU (other streams or
 * threads) race, so serialise them. The first call on a device does the one-time set-up
 * (device address of the array, kernel attributes) and should come before any stream capture.
 * Every call stages a small table from host memory, so a stream that is being captured is
 * refused with MONONN_ERR_INVALID_ARGUMENT. `out` and the row pitches must be 16-byte aligned;
 * a misaligned one is refused on the host, nothing is launched. */
#define MONONN_NOALLOC_MAX_TOKENS 16384
int mononn_attention_noalloc(const void* q, const void* k, const void* v_t, const int32_t* mask,
                             void* out, unsigned batches, unsigned heads, unsigned seq,
                             unsigned ld_qk, unsigned ld_vt, unsigned ld_out, float scale,
                             float mask_scale, int causal, void* cuda_stream);
/* Waits for `cuda_stream`, then reads the status word the kernel keeps in the same static array
 * (no allocation): MONONN_OK, or MONONN_ERR_BARRIER_TIMEOUT when a bounded wait expired during
 * the last mononn_attention_noalloc on this device, in which case `out` is incomplete. Like the
 * entry point itself it has no counterpart in the reference, whose kernels spin without a bound
 * (mononn_engine/core/gpu/synchronization.cc:45-97). */
int mononn_attention_noalloc_status(void* cuda_stream);

void mononn_destroy(mononn_module* m);
const char* mononn_strerror(int code);
/* Message of the last failing call on this thread. */
const char* mononn_last_error(void);

/* TF_MONONN_ENABLED is truthy for "True", "true" or "1"
 * (mononn_engine/helpers/env_variable.cc:20-26); the host shim does not call in otherwise. */
int mononn_enabled(void);

#ifdef __cplusplus
}
#endif
#endif /* MONONN_B200_H_ */
