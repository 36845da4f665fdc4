/*
 * vrb_sharded.h -- C ABI of the multi-GPU host layer (libvrb_sharded.so): one process per GPU, an
 * NCCL communicator owned by the library, the operator kernels of libvrb.so (vrb.h) in between.
 *
 * The reference has no multi-GPU path (its CUDA backend refuses any device but 0,
 * native/src/backend/cuda/cuda_backend.cu:3155), so nothing here replaces a reference interface;
 * what is sharded, and how, follows the operators' own structure:
 *   - DiT operators are independent per token row: token ranges per rank, no entry point needed;
 *   - GroupNorm over a feature map split along H: per-rank shifted moments, ONE all-reduce of
 *     [units, 3] doubles, local normalise (+ SiLU), optional gather of the output;
 *   - the sampler update is flat elementwise: flat ranges, then ONE all-gather of the latent.
 *
 * Every call enqueues on the caller's stream and returns; vrbs_wait() is the bounded wait: it
 * returns when the stream has drained, or -- after the communicator's timeout, or as soon as NCCL
 * reports an asynchronous error -- aborts the communicator (ncclCommAbort) so that no rank hangs on
 * a peer that has gone, and returns VRBS_ERR_TIMEOUT / VRBS_ERR_NCCL.  An aborted communicator
 * refuses further calls; create a new one.
 */
#ifndef VRB_SHARDED_H_
#define VRB_SHARDED_H_

#include <stddef.h>
#include <stdint.h>

#include "vrb.h"

#ifdef __cplusplus
extern "C" {
#endif

typedef struct vrbs_comm vrbs_comm;

typedef enum vrbs_status {
    VRBS_OK = 0,
    VRBS_ERR_INVALID = -1,    /* bad argument */
    VRBS_ERR_KERNEL = -2,     /* an operator entry point of libvrb.so failed; text is its vrb_last_error() */
    VRBS_ERR_CUDA = -3,
    VRBS_ERR_NCCL = -5,       /* NCCL call or asynchronous NCCL error */
    VRBS_ERR_TIMEOUT = -6,    /* vrbs_wait ran out of time: the communicator has been aborted */
    VRBS_ERR_ABORTED = -7     /* the communicator was aborted earlier */
} vrbs_status;

typedef enum vrbs_gather {
    VRBS_GATHER_NONE = 0,     /* out = this rank's normalised slice */
    VRBS_GATHER_NCCL = 1,     /* ncclAllGather into the workspace, then strided placement into out (full tensor) */
    VRBS_GATHER_PEER = 2      /* the normalise kernel stores its slice into every rank's full tensor (destinations) */
} vrbs_gather;

#define VRBS_UNIQUE_ID_BYTES 128

const char* vrbs_last_error(void);
/* Rank 0 makes the id and hands it to the other ranks by whatever channel the launcher has. */
int vrbs_unique_id(void* id128);
/* Communicator on the CURRENT device.  timeout_ms bounds vrbs_wait (<= 0: 30 s). */
int vrbs_create(vrbs_comm** comm, int rank, int world, const void* id128, int timeout_ms);
int vrbs_destroy(vrbs_comm* comm);
int vrbs_rank(const vrbs_comm* comm);
int vrbs_world(const vrbs_comm* comm);
int vrbs_aborted(const vrbs_comm* comm);

/* Scratch for vrbs_group_norm: statistics + (VRBS_GATHER_NCCL) world x local_bytes of staging. 256-byte aligned. */
size_t vrbs_group_norm_workspace_bytes(const vrbs_comm* comm, int64_t batch, int groups, int gather, size_t local_bytes);

/* GroupNorm(groups, eps) [+ SiLU] (CudaBackend::group_norm, cuda_backend.cu:4919-5008, then activation(Silu),
 * native/src/components/autoencoder_kl.cpp:40-41) of x [batch, channels, frames, rows_full, width] split along
 * the rows: x_local is this rank's [batch, channels, frames, rows_local, width] starting at row row0.
 * Statistics are those of the WHOLE tensor: rank 0's first element of every (batch entry, group) is
 * broadcast as the common shift, the shifted moments are all-reduced, every rank finalises the same
 * mean / inverse deviation.  out: the local slice (VRBS_GATHER_NONE) or the full tensor (VRBS_GATHER_NCCL;
 * needs rows_full == world * rows_local); VRBS_GATHER_PEER ignores out and stores into destinations[0..world),
 * full tensors of all ranks mapped into this process (peer memory) -- plain stores, no multicast. */
int vrbs_group_norm(vrbs_comm* comm, const void* x_local, int dtype, const void* weight, int weight_dtype,
                    const void* bias, int bias_dtype, void* out, int64_t batch, int64_t channels, int64_t frames,
                    int64_t rows_local, int64_t rows_full, int64_t row0, int64_t width, int groups, float eps,
                    int fuse_silu, int gather, void* const* destinations, void* workspace, size_t workspace_bytes,
                    vrb_stream stream);

/* cfg_combine + euler_update (vrb_cfg_euler) on this rank's flat range of the replicated latent, then the
 * all-gather of the updated latent into out (count elements; count % (8 * world) == 0). */
int vrbs_cfg_euler(vrbs_comm* comm, const void* sample, const void* unconditional, const void* conditional, void* out,
                   int dtype, int64_t count, float scale, float delta, int subtract_prediction, int guidance_role,
                   int solver_role, vrb_stream stream);

/* Bounded wait for everything enqueued on `stream`; see the header comment. */
int vrbs_wait(vrbs_comm* comm, vrb_stream stream);

/* The watchdog on the host alone (no GPU, no NCCL): a communicator whose peer never joins, so the
 * work never completes.  report = {vrbs_wait's status, milliseconds it took, aborts issued, status of a
 * call made afterwards}. */
int vrbs_watchdog_selftest(int timeout_ms, int64_t* report4);

#ifdef __cplusplus
}
#endif
#endif /* VRB_SHARDED_H_ */
