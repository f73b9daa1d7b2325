/*
 * tnn_b200_plugin — C entry points of the DEVICE_CUDA plug-in (tnn_b200/lib/libtnn_b200_plugin.so) beside what it
 * registers with TNN through static constructors (device, context, blob converter, fused layers, accs, graph pass).
 * A TNN application needs none of them to run a model: TNN::Init / CreateInst / SetInputMat / Forward / GetOutputMat
 * work unchanged.  They exist for tooling (run the graph pass without a GPU, save an optimised model), for serving
 * code that wants page-locked Mats, and for tests (allocation counters, injected allocation failures).
 */
#ifndef TNN_B200_PLUGIN_H_
#define TNN_B200_PLUGIN_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define TNNB200_API __attribute__((visibility("default")))

/* Runs only the graph pass (source/tnn/optimizer/net_optimizer_manager.cc:33-56 would run it inside Instance::Init)
 * on a tnnproto/tnnmodel pair held in memory and writes the fused layer list as text ("Type name in.. -> out..\n").
 * precision: TNN's Precision enum.  Returns the layer count or a negative error.  Needs no GPU. */
TNNB200_API int tnnb200_test_fuse(const char* proto, size_t proto_len, const char* model, size_t model_len, int precision,
                                  char* out, size_t out_cap);
/* The same the way Instance::Init runs it for DEVICE_CUDA (source/tnn/core/instance.cc:86-124): if the pass refuses the
 * graph and fold_constants != 0, the reference's constant folder evaluates the graph's shape arithmetic on DEVICE_NAIVE
 * and the pass runs again.  Layers the folder has evaluated are left out of the listing.  err receives the text of
 * the last refusal (e.g. the layers without a CUDA implementation). */
TNNB200_API int tnnb200_test_fuse_ex(const char* proto, size_t proto_len, const char* model, size_t model_len,
                                     int precision, int fold_constants, char* out, size_t out_cap, char* err,
                                     size_t err_cap);
/* Runs the pass and saves the optimised model with the reference's ModelPacker
 * (source/tnn/interpreter/tnn/model_packer.cc:70-248).  Returns the layer count or a negative error.  Needs no GPU. */
TNNB200_API int tnnb200_fuse_and_pack(const char* proto, size_t proto_len, const char* model, size_t model_len,
                                      int precision, const char* out_proto, const char* out_model);

/* Counters of one GPU's memory arena (the device's allocator; replaces one cudaMalloc per blob,
 * source/tnn/device/cuda/cuda_device.cc:53-64).  out[0] cudaMalloc calls so far, [1] cudaFree calls so far,
 * [2] bytes held from the driver, [3] bytes handed out, [4] live blocks, [5] requests served so far,
 * [6] cudaHostAlloc calls so far (process-wide), [7] page-locked bytes held (process-wide). */
TNNB200_API void tnnb200_arena_stats(int device_id, uint64_t out[8]);
/* Returns wholly free slabs of `device_id` (-1: every GPU) and cached page-locked blocks to the driver; bytes released. */
TNNB200_API uint64_t tnnb200_release_cached_memory(int device_id);
/* Test hook: after `skip` more successful device allocations of the plug-in, the next `count` fail with
 * TNNERR_OUTOFMEMORY (host-side fault injection; count = 0 switches it off). */
TNNB200_API void tnnb200_inject_allocation_failure(int skip, int count);
/* Host-only self-test of the arena's sub-allocation logic (best fit over slabs, merging of freed ranges, the
 * one-allocation-per-block mode with pooled = 0): `steps` seeded random requests and releases against a fake backing
 * store, invariants checked after each.  No CUDA call is made.  Returns 0, or the step at which an invariant broke
 * (message in `err`). */
TNNB200_API int tnnb200_selftest_range_arena(unsigned seed, int steps, int pooled, char* err, int err_cap);

/* The blob converter's host-side conversion (TNN_B200_HOST_CONVERT=1: fp32 host Mats of half-precision blobs are
 * converted on the host cores so that half the bytes cross the bus): src[n] fp32 -> half_out[n] (half_dtype 0 = fp16,
 * 1 = bfloat16 as in tnn_b200.h; round to nearest even, like the device's conversion kernel) and, if back_out is
 * given, back to fp32.  force_scalar = 1 uses the portable scalar code instead of F16C.  No CUDA call is made.
 * Returns 1 if the vector path was used, 0 if the scalar one, negative on bad arguments. */
TNNB200_API int tnnb200_host_convert(const float* src, uint64_t n, int half_dtype, int force_scalar,
                                     uint16_t* half_out, float* back_out);
/* How many Mat <-> blob conversions of this process took the host-side route so far. */
TNNB200_API uint64_t tnnb200_host_conversions(void);

/* CUDA-graph replay counters of the instance that owns `command_queue` (Instance::GetCommandQueue): out[0] Forwards
 * launched layer by layer, [1] captures, [2] graph launches, [3] failed captures / launches (re-run layer by layer).
 * Returns 0, or -1 if the queue belongs to no live instance of the plug-in. */
TNNB200_API int tnnb200_graph_counters(void* command_queue, uint64_t out[4]);

/* Page-locked host memory for Mats (wrap it with Mat(DEVICE_NAIVE, type, dims, ptr)): the blob converter recognises
 * it and makes it the source / target of the DMA itself, with no staging copy on the host.  NULL on failure. */
TNNB200_API void* tnnb200_host_alloc(size_t bytes);
TNNB200_API void  tnnb200_host_free(void* ptr);

#ifdef __cplusplus
}
#endif
#endif /* TNN_B200_PLUGIN_H_ */
