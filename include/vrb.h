/*
 * vrb.h -- C ABI of the B200 (sm_100a) non-GEMM operator library for the vrhino runtime.
 *
 * This is the boundary a vrhino::Backend implementation binds to: every entry point takes
 * raw DEVICE pointers, sizes and a CUDA stream, allocates nothing, never synchronises, launches
 * asynchronously on the given stream and returns 0 or a negative vrb_status (text via
 * vrb_last_error()).  The *_host entry points at the end take HOST pointers instead and stage
 * through device buffers the library owns; they are the only ones that allocate
 * (vrb_device_allocation_count() counts their cudaMalloc calls).
 *
 * Device memory the library's image holds on every GPU that loads it, until the process exits:
 * seven 128 KB function tables (896 KB) used by the bf16 unary kernels on large tensors, and the
 * ~1 MiB scratch of vrb_group_norm_fixed_scratch.  The first large bf16 call per (device,
 * operator) launches a small kernel on the caller's stream that fills the operator's table;
 * vrb_prepare_tables() does that for all of them ahead of time.
 *
 * Each declaration cites the reference interface it replaces; paths are inside the
 * reference project and, when no file is named, mean
 * native/src/backend/cuda/cuda_backend.cu.
 *
 * Dtype codes are the reference's DType enumerators (native/include/vrhino/tensor.h:13).
 * All tensors are dense and contiguous (the reference has no strided tensors).
 */
#ifndef VRB_H_
#define VRB_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define VRB_ABI_VERSION 1

/* enum class DType, native/include/vrhino/tensor.h:13 (the same codes) */
typedef enum vrb_dtype { VRB_F32 = 0, VRB_BF16 = 2, VRB_I64 = 3, VRB_I32 = 4, VRB_U8 = 5 } vrb_dtype;

typedef enum vrb_status {
    VRB_OK = 0,
    VRB_ERR_INVALID = -1,     /* null pointer, non-positive extent, bad enum, illegal broadcast */
    VRB_ERR_UNSUPPORTED = -2, /* dtype / layout combination the reference also rejects */
    VRB_ERR_CUDA = -3,        /* a CUDA runtime call failed; text names it */
    VRB_ERR_WORKSPACE = -4    /* caller's scratch buffer is too small or misaligned */
} vrb_status;

/* enum Activation, native/include/vrhino/backend.h:14 */
typedef enum vrb_activation_kind {
    VRB_SILU = 0, VRB_GELU = 1, VRB_GELU_TANH = 2, VRB_TANH = 3, VRB_RELU = 4
} vrb_activation_kind;

/* binary<Kind>, :3871-3902 */
typedef enum vrb_binary_kind { VRB_ADD = 0, VRB_MUL = 1, VRB_DIV = 2, VRB_MAX = 3 } vrb_binary_kind;

/* QuantType, native/include/vrhino/tensor.h:35 (order of dequantize_kernel<T,Kind>, :641) */
typedef enum vrb_quant_kind { VRB_Q_FP8_E4M3FN = 0, VRB_Q_INT8 = 1, VRB_Q_INT4 = 2 } vrb_quant_kind;

typedef void* vrb_stream; /* cudaStream_t; NULL = the legacy default stream the reference uses */

int vrb_abi_version(void);
/* Text of the calling thread's most recent failure ("" if none). */
const char* vrb_last_error(void);
/* Number of kernels this library has launched in the process (all threads, all streams). */
uint64_t vrb_launch_count(void);
/* Number of device allocations (cudaMalloc) the library has made in the process.  Only the
 * *_host entry points allocate; every other entry point leaves this count unchanged. */
uint64_t vrb_device_allocation_count(void);
/* Fills the current device's function tables (activation kinds, exp, sqrt as bf16 -> bf16 maps,
 * CudaBackend::activation :4179-4188 evaluated on all 65536 inputs) on `stream`: seven small
 * kernels, no allocation, no synchronisation.  Optional -- the operators do it on first use -- but
 * a caller that captures its first launches into a CUDA graph should call it once per device
 * before the capture, otherwise the captured kernels evaluate their tables themselves on every
 * replay (same results, about 10 us slower per launch).  VRB_ERR_INVALID on a capturing stream. */
int vrb_prepare_tables(vrb_stream stream);
/* Overlapped launches (on by default).  The row-norm, gated-residual and table kernels are launched
 * so that the GPU may begin scheduling them while the previous kernel of the stream drains
 * (programmatic dependent launch); each of them waits for that kernel's completion before it
 * touches any caller memory, so results and stream ordering are those of plain launches.  What it
 * buys is the launch gap between short kernels (token shards of a block on 8 GPUs).  0 switches it
 * off (plain launches), non-zero on; returns the previous setting.  Process-wide.  No counterpart
 * in the reference, which launches everything on the legacy default stream. */
int vrb_set_launch_overlap(int enabled);

/* ------------------------------------------------------------------ per-operator forms -- */

/* CudaBackend::add/mul/div/maximum (:3871-3902) on operands already in `dtype`.
 * Shapes broadcast right-aligned, rank <= 8 (:525); out has the broadcast shape. */
int vrb_binary(int kind, const void* a, const int64_t* a_shape, int a_rank,
               const void* b, const int64_t* b_shape, int b_rank,
               void* out, int dtype, vrb_stream stream);

/* CudaBackend::cast (:3978) / the conversion kernels :597-628.  src dtype may be VRB_U8. */
int vrb_cast(const void* src, int src_dtype, void* dst, int dst_dtype, int64_t count,
             vrb_stream stream);

/* CudaBackend::activation (:4179-4188), clamp (:5128), exp, sqrt (:5134-5173). */
int vrb_activation(int kind, const void* x, void* out, int dtype, int64_t count, vrb_stream stream);
int vrb_clamp(const void* x, void* out, int dtype, int64_t count, float minimum, float maximum,
              vrb_stream stream);
int vrb_exp(const void* x, void* out, int dtype, int64_t count, vrb_stream stream);
int vrb_sqrt(const void* x, void* out, int dtype, int64_t count, vrb_stream stream);

/* CudaBackend::layer_norm (:4057-4089).  Output dtype = x's.  weight/bias may be NULL; they
 * may be given in F32 or BF16 and are converted to x's dtype as the reference does. */
int vrb_layer_norm(const void* x, int dtype, const void* weight, int weight_dtype,
                   const void* bias, int bias_dtype, void* out,
                   int64_t rows, int64_t width, float eps, vrb_stream stream);

/* CudaBackend::rms_norm over the last axis (:4091-4160).  out_dtype = x_dtype, or F32 for
 * BF16 input (needs a weight, :4123).  weight is converted to out_dtype. */
int vrb_rms_norm(const void* x, int x_dtype, const void* weight, int weight_dtype,
                 void* out, int out_dtype, int64_t rows, int64_t width, float eps,
                 vrb_stream stream);

/* CudaBackend::rms_norm over an inner axis (:4161-4176): x is [outer, axis, inner]. */
int vrb_rms_norm_axis(const void* x, int dtype, const void* weight, int weight_dtype, void* out,
                      int64_t outer, int64_t axis, int64_t inner, float eps, int fuse_silu,
                      vrb_stream stream);

/* CudaBackend::pixel_norm (:5048-5086) over the middle axis of x [outer, channels, inner]:
 *   y = x / sqrtf(mean_c(x^2) + eps)  in x's dtype, the kernels' F32 summation schedules (:2097-2165).
 * With scale / shift ([outer, channels], both or neither) the result continues as the head of LTX's
 * decoder_residual (native/src/architectures/ltx.cpp:221-227):
 *   out = cast(F32(y) * (1 + F32(scale)) + F32(shift), out_dtype)     modulate, common.cpp:51-61
 * and with fuse_silu the activation (activation(Silu)) is applied before the final cast.
 * Without scale / shift out_dtype must equal dtype. */
int vrb_pixel_norm(const void* x, int dtype, const void* scale, const void* shift, int mod_dtype,
                   int fuse_silu, void* out, int out_dtype, int64_t outer, int64_t channels,
                   int64_t inner, float eps, vrb_stream stream);

/* The shared-memory tile kernels (vrb_pixel_norm, vrb_l2_normalize, vrb_rms_norm_axis) load their tiles with tensor-map copies
 * (cp.async.bulk.tensor, completion on an mbarrier) where the geometry allows.  vrb_set_tensor_map_tiles(0) makes them
 * use per-thread 16-byte asynchronous copies instead (same shared-memory layout, same results); returns the previous
 * setting.  Every wait on such a copy is bounded: a kernel whose wait runs out sets a flag in device memory and
 * returns; vrb_async_wait_failures reads the flag (a synchronising copy; 0 = no wait has ever run out on the current
 * device). */
int vrb_set_tensor_map_tiles(int enabled);
int vrb_async_wait_failures(int* failures);

/* CudaBackend::l2_normalize (:5088-5110, l2_normalize_kernel :1142-1176) over the middle axis of
 * x [outer, channels, inner]:  y = x / (sqrtf(sum_c(x^2)) + eps)  in x's dtype; eps >= 0.  Same tiles and
 * F32 summation as vrb_pixel_norm (the reference's 256-thread tree adds the same squares in another
 * order: results agree to the last bits of the sum). */
int vrb_l2_normalize(const void* x, void* out, int dtype, int64_t outer, int64_t channels, int64_t inner,
                     float eps, vrb_stream stream);

/* ---- layout operators -------------------------------------------------------------------------
 * Shapes are arrays of `rank` extents (rank <= 8), outermost first; tensors are contiguous; dtype is
 * VRB_F32 or VRB_BF16; results are bit-exact copies.  A tensor with a zero extent launches nothing.
 *
 * CudaBackend::permute (:3936-3947, permute_kernel :767-780): out has shape[dims[d]] along d and
 * out[c_0..c_{r-1}] = x[the coordinate whose axis dims[d] is c_d].  "Invalid permutation" unless dims is
 * a permutation of 0..rank-1. */
int vrb_permute(const void* x, void* out, int dtype, int rank, const int64_t* shape, const int64_t* dims,
                vrb_stream stream);

/* CudaBackend::slice (:3960-3970, slice_kernel :782-796): x[..., start:stop, ...] along `dim` of `shape`
 * (x's shape).  As there: a negative dim counts from the end, negative start / stop are offset by the
 * extent, start is clamped into [0, extent] and stop into [start, extent]; out must hold the clamped
 * range. */
int vrb_slice(const void* x, void* out, int dtype, int rank, const int64_t* shape, int dim, int64_t start,
              int64_t stop, vrb_stream stream);

/* CudaBackend::concat (:3949-3958, copy_into_concat_kernel :798-813): `count` tensors that differ only
 * along `dim`, where input k has extents[k]; `shape` is the OUTPUT's shape and shape[dim] must equal the
 * sum of extents ("concat shape mismatch" otherwise).  One launch per input, like the reference. */
int vrb_concat(const void* const* inputs, const int64_t* extents, int count, void* out, int dtype, int rank,
               const int64_t* shape, int dim, vrb_stream stream);

/* CudaBackend::pad (:4875-4883, pad_kernel :1771-1788): out has shape[d] + before[d] + after[d] along
 * every axis (per-axis arrays of `rank` entries; the reference's innermost-first pair vector is unpacked
 * by the caller).  replicate == 0: positions outside x hold `value` rounded to dtype; replicate != 0:
 * the nearest element of x (coordinates clamped per axis).  "Negative padding unsupported". */
int vrb_pad(const void* x, void* out, int dtype, int rank, const int64_t* shape, const int64_t* before,
            const int64_t* after, float value, int replicate, vrb_stream stream);

/* Two pads of the reference in one pass: per axis d, replicate_axes[d] != 0 replicates, 0 fills with `value`; an
 * element outside the source along ANY constant-mode axis holds `value`, as if the replicate axes had been padded
 * first and the constant axes afterwards.  That is LTX's edge_time_conv (native/src/architectures/ltx.cpp:205-215):
 * pad(x, {0,0,0,0,t,t}, 0, Replicate) followed by pad(., {w,w,h,h}, 0) before every convolution. */
int vrb_pad_axes(const void* x, void* out, int dtype, int rank, const int64_t* shape, const int64_t* before,
                 const int64_t* after, float value, const int* replicate_axes, vrb_stream stream);

/* CudaBackend::interpolate_nearest (:5010-5016, interpolate_kernel :2033-2045): out[c] = x[floor(c_d * in_shape[d] /
 * out_shape[d]) along every axis d]; the caller computes out_shape (the reference: floor(extent * factor) on the
 * trailing axes).  At most three axes may differ between the shapes, and they must be the trailing ones after any
 * number of equal leading axes.  The Wan VAE's 2x spatial upsampling (wan.cpp:268) takes a form that reads 16 bytes
 * and writes them doubled into both output rows. */
int vrb_interpolate_nearest(const void* x, void* out, int dtype, int rank, const int64_t* in_shape,
                            const int64_t* out_shape, vrb_stream stream);

/* CudaBackend::indexed_gather (:3981-4055, indexed_gather_kernel :1754-1768): out [batches, indices_per_batch, width] =
 * table [batches, rows, width] gathered along rows by indices [batches, indices_per_batch] (index_dtype VRB_I64 or
 * VRB_I32, on the device).  batches == 0: one table [rows, width] for all indices_per_batch indices.  The caller
 * validates 0 <= index < rows beforehand (the reference does so on the host and raises "indexed_gather index out of
 * range"); a row with an index out of range is left unwritten. */
int vrb_indexed_gather(const void* table, const void* indices, int index_dtype, void* out, int dtype, int64_t batches,
                       int64_t rows, int64_t width, int64_t indices_per_batch, vrb_stream stream);

/* CudaBackend::softmax (:4893-4917, softmax_axis_kernel :1808-1829) over the middle axis of x [outer, axis, inner]:
 * maximum, then the sum of expf(x - max) accumulated in F32 in index order (the reference's order: same bits), then
 * expf(x - max) / sum stored in x's dtype. */
int vrb_softmax(const void* x, void* out, int dtype, int64_t outer, int64_t axis, int64_t inner, vrb_stream stream);

/* CudaBackend::rng_normal (:5120-5126, rng_normal_kernel :2225-2231): out[i] = the first normal of cuRAND's
 * Philox4x32-10 stream (seed, subsequence i, offset), F32 or rounded to bf16: the reference's values bit for bit.
 * The caller keeps the RngState (native/include/vrhino/backend.h:17-21) and adds 4 to its offset after every call. */
int vrb_rng_normal(void* out, int dtype, int64_t count, uint64_t seed, uint64_t offset, vrb_stream stream);

/* CudaBackend::reduce_sum (:4885-4892, reduce_sum_kernel :1790-1806) over the middle axis of x [outer, reduced, inner]:
 * out[o, i] = sum of x[o, r, i] for r = 0, 1, ... in that order, accumulated in F32 and stored in x's dtype (the
 * reference's order, so the same bits).  reduced == 0 gives zeros. */
int vrb_reduce_sum(const void* x, void* out, int dtype, int64_t outer, int64_t reduced, int64_t inner,
                   vrb_stream stream);

/* CudaBackend::sinusoidal_embedding (:4190-4196, sinusoidal_kernel :1178-1198): positions [count] ->
 * out [count, width].  half = width / 2; logical column l = flip ? (column + half) % (2 half) : column;
 * out = (l < half ? sin : cos)(position * exp(-ln(10000) * (l % half) / (half - downscale))); an odd last
 * column is 0.  frequency_f64 != 0 evaluates in double and rounds once; otherwise every step is single
 * precision, in the reference kernel's order. */
int vrb_sinusoidal_embedding(const void* positions, void* out, int dtype, int64_t count, int64_t width,
                             int flip, double downscale, int frequency_f64, vrb_stream stream);

/* CudaBackend::pixel_shuffle_nd (:5112-5118, pixel_shuffle_kernel :2170-2186):
 * x [batch, channels*ft*fh*fw, frames, height, width] -> out [batch, channels, frames*ft, height*fh, width*fw],
 * out[b, c, t*ft+pt, h*fh+ph, w*fw+pw] = x[b, ((c*ft+pt)*fh+ph)*fw+pw, t, h, w]. */
int vrb_pixel_shuffle(const void* x, void* out, int dtype, int64_t batch, int64_t channels,
                      int64_t frames, int64_t height, int64_t width, int factor_t, int factor_h,
                      int factor_w, vrb_stream stream);

/* LTX depth_to_space (native/src/architectures/ltx.cpp:250-259) after its convolution, in one pass:
 * projected [batch, 4*C, T, H, W] (the convolution output), input [batch, C, T, H, W] ->
 *   out = slice(pixel_shuffle(projected, {2,2,2}), 2, 1, 2T)
 *       + slice(concat(4 x pixel_shuffle(input, {2,2,2}), 1), 2, 1, 2T)        [batch, C/2, 2T-1, 2H, 2W]
 * all tensors in `dtype`; C a multiple of 8. */
int vrb_depth_to_space_residual(const void* projected, const void* input, void* out, int dtype,
                                int64_t batch, int64_t input_channels, int64_t frames,
                                int64_t height, int64_t width, vrb_stream stream);

/* CudaBackend::rope_nd (:4198-4213).  cos/sin have f_shape and broadcast against x_shape. */
int vrb_rope(const void* x, int x_dtype, const int64_t* x_shape, int x_rank,
             const void* cosine, const void* sine, int f_dtype, const int64_t* f_shape, int f_rank,
             void* out, vrb_stream stream);

/* copy_to_device, quantized branch (:3214-3296): packed [rows, inner] with scales
 * [rows, ceil(inner/group_size)] -> out_dtype.  FP8 decode :630-638. */
int vrb_dequantize(int kind, const void* packed, const float* scales, void* out, int out_dtype,
                   int64_t rows, int64_t inner, int64_t group_size, vrb_stream stream);

/* CudaBackend::group_norm (:4919-5008) on x [batch, channels, spatial], optionally followed by
 * the SiLU the VAE call sites apply next (native/src/components/autoencoder_kl.cpp:40-41).
 * workspace: vrb_group_norm_workspace_bytes() bytes of device scratch, 256-byte aligned. */
size_t vrb_group_norm_workspace_bytes(int64_t batch, int groups);
int vrb_group_norm(const void* x, int dtype, const void* weight, int weight_dtype,
                   const void* bias, int bias_dtype, void* out,
                   int64_t batch, int64_t channels, int64_t spatial, int groups, float eps,
                   int fuse_silu, void* workspace, size_t workspace_bytes, vrb_stream stream);

/* Per-frame GroupNorm of a video feature map without the two permutes: x and out are
 * [batch, channels, frames, spatial]; statistics per (batch entry, frame, group), i.e. what
 * frame_group_norm (native/src/architectures/mochi.cpp:365-371) computes by permuting to
 * [batch*frames, channels, spatial], calling group_norm and permuting back.  Needs spatial % 8 == 0,
 * 16-byte aligned tensors and channels/groups <= 64 (VRB_ERR_UNSUPPORTED otherwise: permute and
 * call vrb_group_norm).  workspace: vrb_group_norm_frames_workspace_bytes() bytes, 256-byte aligned. */
size_t vrb_group_norm_frames_workspace_bytes(int64_t batch, int64_t frames, int groups);
int vrb_group_norm_frames(const void* x, int dtype, const void* weight, int weight_dtype,
                          const void* bias, int bias_dtype, void* out,
                          int64_t batch, int64_t channels, int64_t frames, int64_t spatial, int groups,
                          float eps, int fuse_silu, void* workspace, size_t workspace_bytes, vrb_stream stream);

/* vrb_group_norm without a caller-provided workspace.  This entry point has no counterpart in
 * the reference (whose operators take scratch from the backend's own temporary pool); it exists
 * for callers that cannot hand over device scratch: a backend whose device budget is entirely
 * owned by a memory planner, so nothing may be allocated once a step is running, or a host
 * thread that must stay out of cudaMalloc because that call synchronises the device.
 * The scratch is a fixed array inside the library's device image: each GPU that loads the
 * library holds about 1 MiB for it until the process exits, and it limits the call to
 * batch * groups <= VRB_GROUP_NORM_FIXED_SCRATCH_MAX_UNITS; larger problems are refused with
 * VRB_ERR_WORKSPACE and must use vrb_group_norm.  No memory is allocated or freed, here or in
 * anything it calls (the SiLU table of the bf16 + fuse_silu path is part of the library's device
 * image as well).  The first call on a device looks up the array's device address (one runtime
 * query with that device current; the address is kept per device index and does not survive
 * cudaDeviceReset) and, for bf16 + fuse_silu on large tensors, launches the table-fill kernel
 * ahead of the operator's own; make that first call before any stream capture begins.  All calls on a device share the one array, which keeps whatever the previous call
 * wrote; this operator overwrites every slot it later reads, so nothing needs clearing, but
 * two calls whose kernels can overlap on the GPU (different streams, no ordering between them)
 * race on it -- order them on one stream or with events. */
#define VRB_GROUP_NORM_FIXED_SCRATCH_MAX_UNITS 1024
int vrb_group_norm_fixed_scratch(const void* x, int dtype, const void* weight, int weight_dtype,
                                 const void* bias, int bias_dtype, void* out,
                                 int64_t batch, int64_t channels, int64_t spatial, int groups, float eps,
                                 int fuse_silu, vrb_stream stream);

/* The two halves of vrb_group_norm for a tensor whose spatial axis is split over ranks:
 * moments[unit] = {n, sum(x - shift[unit]), sum((x - shift[unit])^2)} as three doubles per
 * unit over this rank's slice; slices add; vrb_group_norm_finalize turns the added moments
 * into mean / inverse-stddev; vrb_group_norm_apply normalises a slice.
 * x is [batch, channels, spatial_local]. */
int vrb_group_norm_moments(const void* x, int dtype, int64_t batch, int64_t channels,
                           int64_t spatial_local, int groups, const float* shift,
                           double* moments, void* workspace, size_t workspace_bytes,
                           vrb_stream stream);
int vrb_group_norm_finalize(const double* moments, const float* shift, int64_t units, float eps,
                            float* mean, float* inverse, vrb_stream stream);
int vrb_group_norm_apply(const void* x, int dtype, const void* weight, int weight_dtype,
                         const void* bias, int bias_dtype, void* out,
                         int64_t batch, int64_t channels, int64_t spatial_local, int groups,
                         const float* mean, const float* inverse, int fuse_silu,
                         vrb_stream stream);

/* vrb_group_norm_apply whose stores do the all-gather of an H-sharded feature map: x is this
 * rank's slice [batch, channels, frames, spatial_local] (spatial_local = local rows x row width);
 * every destination is a FULL tensor [batch, channels, frames, spatial_full] -- this GPU's own and
 * the peer-mapped ones of the other ranks -- and receives the slice at element offset
 * spatial_offset of every (batch entry, channel, frame) plane.  mean / inverse are per
 * (batch entry, group) as vrb_group_norm_finalize produced them from the all-reduced moments.
 * Plain st.global to the peer pointers; the caller orders the ranks on both sides: before the
 * launch every rank must be done reading the previous contents of its destination, and after it
 * every rank's stores must have landed before anyone reads (any collective or barrier on the
 * stream does either).  spatial_local, spatial_full and spatial_offset must be multiples
 * of 8 elements.  No counterpart in the reference, which has no multi-GPU path. */
int vrb_group_norm_apply_scatter(const void* x, int dtype, const void* weight, int weight_dtype,
                                 const void* bias, int bias_dtype, void* const* destinations, int destination_count,
                                 int64_t batch, int64_t channels, int64_t frames, int64_t spatial_local,
                                 int64_t spatial_full, int64_t spatial_offset, int groups,
                                 const float* mean, const float* inverse, int fuse_silu, vrb_stream stream);

/* ------------------------------------------------------------------------ fused chains -- */
/* Each fused form produces what the cited chain of separate reference kernels produces,
 * including every intermediate rounding, while reading each tensor once. */

/* gated_residual / residual_add (common.cpp:134-144) followed by the LayerNorm the block applies
 * to the updated stream next, with or without adaLN modulation (wan.cpp:95-110), in one pass:
 *   state_out = residual + branch * gate          (gate NULL: residual + branch), in state_dtype
 *   out       = cast(modulate(layer_norm(state_out, weight, bias, eps), shift, scale), out_dtype)
 *               (scale NULL: cast(layer_norm(...), out_dtype))
 * Every rounding of the unfused chain is kept.  One kernel when the stream is BF16 throughout
 * (each tensor crosses HBM once: 8 B per element instead of 6 + 4); other dtype contracts run
 * the two operators one after the other.  gate is [gate_vectors, width], scale / shift
 * [mod_vectors, width]. */
int vrb_gated_residual_layer_norm_modulate(
    const void* residual, int residual_dtype, const void* branch, int branch_dtype,
    const void* gate, int gate_dtype, int64_t gate_rows_per_vector, int64_t gate_vectors,
    void* state_out, int state_dtype,
    const void* weight, int weight_dtype, const void* bias, int bias_dtype,
    const void* scale, const void* shift, int mod_dtype, int64_t rows_per_vector, int64_t mod_vectors,
    void* out, int out_dtype, int64_t rows, int64_t width, float eps, vrb_stream stream);

/* The same merge for the LTX block, whose next norm is RMSNorm without a weight
 * (native/src/architectures/ltx.cpp:100-151; ltx_self_attention_graph.cpp:30-44):
 *   state = vrb_gated_residual(residual, branch, gate);  out = vrb_rms_norm_modulate(state, scale, shift). */
int vrb_gated_residual_rms_norm_modulate(const void* residual, int residual_dtype,
                                         const void* branch, int branch_dtype,
                                         const void* gate, int gate_dtype,
                                         int64_t gate_rows_per_vector, int64_t gate_vectors,
                                         void* state_out, int state_dtype,
                                         const void* scale, const void* shift, int mod_dtype,
                                         int64_t rows_per_vector, int64_t mod_vectors,
                                         void* out, int out_dtype, int64_t rows, int64_t width,
                                         float eps, vrb_stream stream);

/* layer_norm (:4057) -> modulate (native/src/architectures/common.cpp:51-61) -> cast to
 * out_dtype (the consumer cast, :3674).  scale/shift are [mod_vectors, width]; row r uses
 * vector (r / rows_per_vector) % mod_vectors.  shift may be NULL.  weight/bias may be NULL. */
int vrb_layer_norm_modulate(const void* x, int x_dtype, const void* weight, int weight_dtype,
                            const void* bias, int bias_dtype,
                            const void* scale, const void* shift, int mod_dtype,
                            int64_t rows_per_vector, int64_t mod_vectors,
                            void* out, int out_dtype, int64_t rows, int64_t width, float eps,
                            vrb_stream stream);

/* layer_norm (:4057) -> cast to out_dtype: the F32-residual policy's norm3 feeding the
 * cross-attention projections (native/src/architectures/wan.cpp:98-104), whose linear
 * converts its F32 operand to BF16 (:3674). */
int vrb_layer_norm_cast(const void* x, int x_dtype, const void* weight, int weight_dtype,
                        const void* bias, int bias_dtype, void* out, int out_dtype,
                        int64_t rows, int64_t width, float eps, vrb_stream stream);

/* rms_norm(x, no weight, eps) (:4091) -> modulate (common.cpp:51-61) -> cast: the LTX block
 * (native/src/architectures/ltx_self_attention_graph.cpp:30-44). */
int vrb_rms_norm_modulate(const void* x, int x_dtype, const void* scale, const void* shift,
                          int mod_dtype, int64_t rows_per_vector, int64_t mod_vectors,
                          void* out, int out_dtype, int64_t rows, int64_t width, float eps,
                          vrb_stream stream);

/* rms_norm(x, no weight, eps) * (1 + scale) multiplied in x's dtype:
 * native/src/architectures/mochi.cpp:230-231.  out dtype = x's. */
int vrb_rms_norm_scale(const void* x, int dtype, const void* scale, int scale_dtype,
                       int64_t rows_per_vector, int64_t mod_vectors,
                       void* out, int64_t rows, int64_t width, float eps, vrb_stream stream);

/* attention_norm (common.cpp:62-68: rms_norm widened to F32) -> operation_rope
 * (common.cpp:69-76) -> cast to out_dtype (operation_attention, common.cpp:77-87).
 * norm_width is the normalised extent: `width` (Wan: whole model dim, then head split) or
 * the head width (Mochi / Hunyuan per-head norm); rows*width/norm_width rows are normalised.
 * cos/sin: F32 [f_rows, f_width] with f_width dividing width; element (row r, column c)
 * uses table row (r / rows_per_f_row) % f_rows, column c % f_width.  cosine may be NULL
 * (norm + cast only: the cross-attention q/k of native/src/architectures/wan.cpp:38-46). */
int vrb_rms_norm_rope(const void* x, int x_dtype, const void* weight, int weight_dtype,
                      const void* cosine, const void* sine, int64_t f_rows, int64_t f_width,
                      int64_t rows_per_f_row, void* out, int out_dtype,
                      int64_t rows, int64_t width, int64_t norm_width, float eps,
                      vrb_stream stream);

/* vrb_rms_norm_rope with cos / sin tables in `table_dtype` (F32 or BF16; rope_kernel :1200-1215 widens
 * BF16 frequencies exactly): the LTX graph keeps its tables in the execution dtype
 * (native/src/architectures/ltx_self_attention_graph.cpp:52-54). */
int vrb_rms_norm_rope_tables(const void* x, int x_dtype, const void* weight, int weight_dtype,
                             const void* cosine, const void* sine, int table_dtype, int64_t f_rows,
                             int64_t f_width, int64_t rows_per_f_row, void* out, int out_dtype,
                             int64_t rows, int64_t width, int64_t norm_width, float eps, vrb_stream stream);

/* vrb_rms_norm_rope_tables on TWO tensors in one launch: the q and k projections of an attention block
 * (native/src/architectures/wan.cpp:38-52 normalises and rotates q, then k; the cross-attention q and
 * its text-token k at :38-46 are the cosine == NULL form with different row counts).  Both share
 * dtypes, widths, eps and tables; each has its own tensor, norm weight and row count, and row r of
 * either uses table row (r / rows_per_f_row) % f_rows.  Results are bit-identical to two calls of
 * vrb_rms_norm_rope_tables; what is saved is a launch, and the tables are fetched from HBM once. */
int vrb_rms_norm_rope_pair(const void* x_a, const void* weight_a, void* out_a, int64_t rows_a,
                           const void* x_b, const void* weight_b, void* out_b, int64_t rows_b,
                           int x_dtype, int weight_dtype, const void* cosine, const void* sine, int table_dtype,
                           int64_t f_rows, int64_t f_width, int64_t rows_per_f_row, int out_dtype,
                           int64_t width, int64_t norm_width, float eps, vrb_stream stream);

/* gated_residual (common.cpp:139-144) and, with gate == NULL, residual_add (:134-138):
 * out = T(residual) + round_T(T(branch) * T(gate)), T = state_dtype.  gate is
 * [gate_vectors, width]; row r uses vector (r / rows_per_vector) % gate_vectors. */
int vrb_gated_residual(const void* residual, int residual_dtype, const void* branch, int branch_dtype,
                       const void* gate, int gate_dtype, int64_t rows_per_vector, int64_t gate_vectors,
                       void* out, int state_dtype, int64_t rows, int64_t width, vrb_stream stream);

/* normalized_gated_residual (mochi.cpp:204-211) with the gate already bounded by tanh:
 * out = T(residual) + round_T(T(rms_norm(branch, none, eps)) * T(gate)). */
int vrb_rms_norm_gated_residual(const void* residual, int residual_dtype,
                                const void* branch, int branch_dtype,
                                const void* gate, int gate_dtype,
                                int64_t rows_per_vector, int64_t gate_vectors,
                                void* out, int state_dtype, int64_t rows, int64_t width,
                                float eps, vrb_stream stream);

/* The Mochi block's residual update and the pre-norm of the layer that follows it, in one pass
 * (native/src/architectures/mochi.cpp:204-211 then :228-231):
 *   state_out = vrb_rms_norm_gated_residual(residual, branch, gate', branch_eps),  gate' = tanh(gate) if gate_tanh
 *               (activation(gate, Tanh) in the gate's dtype, as the block computes it) else gate
 *   out       = vrb_rms_norm_scale(state_out, scale, eps)                          in the stream's dtype
 * One kernel when residual, branch and the updated stream are BF16 (each tensor crosses HBM once: 8 B
 * per element instead of 6 + 4, and the tanh of the [vectors, width] gate costs no launch); other dtype
 * contracts run the two operators (then gate_tanh must be 0: apply vrb_activation to the gate first). */
int vrb_rms_norm_gated_residual_rms_norm_scale(
    const void* residual, int residual_dtype, const void* branch, int branch_dtype, float branch_eps,
    const void* gate, int gate_dtype, int gate_tanh, int64_t gate_rows_per_vector, int64_t gate_vectors,
    void* state_out, int state_dtype, const void* scale, int scale_dtype, int64_t rows_per_vector, int64_t scale_vectors,
    void* out, int64_t rows, int64_t width, float eps, vrb_stream stream);

/* ---- the bf16 linear's epilogue and the operator that reads its result --------------------
 * CudaBackend::linear (native/src/backend/cuda/cuda_backend.cu:3661-3866) leaves the GEMM result in an
 * F32 accumulation buffer [rows, width] and runs fused_bf16_linear_output_kernel (:754-764, called
 * at :3831 and :3846):  y = bf16(accumulation + float(bias)),  bias bf16 [width] or NULL.
 * vrb_linear_output is that kernel.  The three forms below also apply the operator the DiT
 * blocks run on y next, so y itself is never written; each keeps every rounding of the separate
 * kernels (results are bit-identical to vrb_linear_output followed by the named entry point). */
int vrb_linear_output(const float* accumulation, const void* bias, void* out, int64_t rows,
                      int64_t width, vrb_stream stream);
/* out = activation(kind, y) as bf16   (wan.cpp:109-112: linear -> activation(GeluTanh)) */
int vrb_linear_output_activation(const float* accumulation, const void* bias, int kind, void* out,
                                 int64_t rows, int64_t width, vrb_stream stream);
/* out = vrb_gated_residual(residual, y, gate)   (wan.cpp:114-116: linear -> gated_residual;
 * gate NULL = residual_add, wan.cpp:99-103) */
int vrb_linear_output_gated_residual(const float* accumulation, const void* bias,
                                     const void* residual, int residual_dtype,
                                     const void* gate, int gate_dtype,
                                     int64_t rows_per_vector, int64_t gate_vectors,
                                     void* out, int state_dtype, int64_t rows, int64_t width,
                                     vrb_stream stream);
/* accumulation [rows, 2*hidden], bias [2*hidden]: out = vrb_swiglu(y) as bf16 [rows, hidden]
 * (mochi.cpp:195-202) */
int vrb_linear_output_swiglu(const float* accumulation, const void* bias, void* out, int64_t rows,
                             int64_t hidden, vrb_stream stream);

/* SamplingPrimitives::linear_combine (native/src/sampling/sampling.cpp:173-179) in one pass, 1..4 terms:
 *   out = ((v0 (x) c0  +  v1 (x) c1)  +  v2 (x) c2)  + ...
 * (x) = precision_scalar_binary (native/src/precision/precision.cpp:196-223): scalar_role != 0 -> F32 product
 * rounded to `dtype`; 0 -> coefficient rounded to `dtype` first; + = one add in `dtype`.
 * v_to_x0 (:204-214) and affine_first_order (:229-239) are its two-term forms. */
int vrb_linear_combine(const void* const* values, const float* coefficients, int terms, void* out,
                       int dtype, int64_t count, int scalar_role, vrb_stream stream);

/* SwiGLU (mochi.cpp:195-202) without the two slice copies: projected is [rows, 2*hidden],
 * out[r, j] = round(projected[r, j] * round(silu(projected[r, hidden + j]))). */
int vrb_swiglu(const void* projected, void* out, int dtype, int64_t rows, int64_t hidden,
               vrb_stream stream);

/* SamplingPrimitives::cfg_combine (native/src/sampling/sampling.cpp:181-183).
 * scalar_role != 0: the guidance coefficient has a declared scalar role, so each multiply is
 * done in F32 and rounded to `dtype` (native/src/precision/precision.cpp:196-223);
 * 0: legacy, the coefficient itself is rounded to `dtype` first. */
int vrb_cfg_combine(const void* unconditional, const void* conditional, void* out, int dtype,
                    int64_t count, float scale, int scalar_role, vrb_stream stream);

/* SamplingPrimitives::euler_update (sampling.cpp:185-193): out = sample + prediction *
 * (delta * (subtract ? -1 : 1)) with the reference's rounding of each product.  delta is the
 * value the one-element coefficient tensor holds (a caller whose execution dtype is BF16 and
 * whose policy declares no solver role passes the BF16-rounded delta, as the reference's
 * host-scalar multiply produces). */
int vrb_euler_update(const void* sample, const void* prediction, void* out, int dtype,
                     int64_t count, float delta, int subtract_prediction, int scalar_role,
                     vrb_stream stream);

/* SamplingPrimitives::flow_to_x0 (sampling.cpp:200-202): out = sample + output * (-sigma). */
int vrb_flow_to_x0(const void* sample, const void* model_output, void* out, int dtype,
                   int64_t count, float sigma, int scalar_role, vrb_stream stream);

/* cfg_combine followed by euler_update on its result, one pass (sampling.cpp:465-477).
 * guided (optional, may be NULL) receives the cfg_combine result. */
int vrb_cfg_euler(const void* sample, const void* unconditional, const void* conditional,
                  void* guided, void* out, int dtype, int64_t count, float scale, float delta,
                  int subtract_prediction, int guidance_role, int solver_role, vrb_stream stream);

/* ---------------------------------------------------------------- host-buffer entry points -- */
/* The reference's operators accept host tensors and upload them on demand (copy_to_device,
 * :3195); results come back through copy_to_host.  These forms do the same for whole fused
 * chains: every pointer is a HOST pointer.  Rows are cut into blocks and streamed through
 * device buffers the library owns on three streams, so upload, kernel and download overlap;
 * operands shared by all rows (vectors of `width`, the norm weight) are uploaded once.
 * Full overlap needs page-locked host buffers (cudaMallocHost / cudaHostRegister).
 * Synchronous: when a call returns -- with success or with an error -- no copy to or from the
 * caller's buffers is in flight, and on success `out` holds the result.  Buffers and streams are
 * kept per device (the device current at the call).  These are the only entry points that allocate
 * device memory; vrb_host_release() frees the current device's. */

/* vrb_layer_norm_modulate on host buffers; scale == NULL gives vrb_layer_norm_cast. */
int vrb_host_layer_norm_modulate(const void* x, int x_dtype, const void* weight, int weight_dtype,
                                 const void* bias, int bias_dtype, const void* scale, const void* shift,
                                 int mod_dtype, void* out, int out_dtype,
                                 int64_t rows, int64_t width, float eps);
/* vrb_rms_norm_rope on host buffers; cos / sin are F32 [rows, f_width] (one table row per token,
 * f_width dividing width) or NULL. */
int vrb_host_rms_norm_rope(const void* x, int x_dtype, const void* weight, int weight_dtype,
                           const void* cosine, const void* sine, int64_t f_width,
                           void* out, int out_dtype, int64_t rows, int64_t width, int64_t norm_width,
                           float eps);
/* vrb_gated_residual on host buffers with one gate vector [width] (or NULL). */
int vrb_host_gated_residual(const void* residual, int residual_dtype, const void* branch, int branch_dtype,
                            const void* gate, int gate_dtype, void* out, int state_dtype,
                            int64_t rows, int64_t width);
/* vrb_activation on a host tensor viewed as [rows, width]. */
int vrb_host_activation(int kind, const void* x, void* out, int dtype, int64_t rows, int64_t width);
void vrb_host_release(void);

#ifdef __cplusplus
}
#endif
#endif /* VRB_H_ */
