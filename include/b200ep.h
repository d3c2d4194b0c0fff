/* b200ep - expert-parallel MoE layer over peer memory (NVLink / NVSwitch), no Python and
 * no collective library on the data path.
 *
 * Only the MoE layer shards (expert e lives on rank e / (ne / world)); the activations
 * x [T, d] are replicated and the output comes back replicated.  The reference has no
 * expert parallelism to compare with (its one collective is the data-parallel gradient
 * all-reduce, training/distributed.cpp:187-308); the layer's arithmetic is the single-GPU
 * layer's (core/moe_cpu.cpp:198-288) cut at its exchange points (b200_moe_route /
 * _dispatch_pack / _experts_rows / _shared_expert / _combine of b200ops.h), so routing
 * indices and the slot order are bit-identical to one GPU and the result is run-to-run
 * bit-stable.
 *
 * One process per GPU.  Every rank allocates one block of device memory with the same
 * layout (receive rows, returned results, replicated output, headers, flags) and maps its
 * peers' blocks (CUDA IPC across processes; plain pointers for ranks of one process).
 * A forward pass is, per rank, stream-ordered and free of host synchronisation:
 *
 *   route + dispatch  this rank's token slice [rank T / world, (rank + 1) T / world): top-K and the
 *                     expert-sorted order of its (token, k) slots; one kernel rounds each slot's
 *                     row to fp16 and stores it straight into the block of the rank that owns its
 *                     expert, with a header (rows per local expert, where they sit in the sender's
 *                     order), fences, and raises the sender's flag there (the pass number); the
 *                     shared expert of the slice runs meanwhile on a second stream
 *   experts + return  waits (bounded) for every sender's flag, turns the headers into a group list
 *                     (gaps between the senders' regions are skipped by the tile scheduler), runs
 *                     the grouped tcgen05 GEMMs over (sender, local expert) blocks in arrival order;
 *                     the down projection's epilogue stores each result row at its home in the
 *                     sender's block; fence, flag
 *   combine + gather  waits for the returns, adds shared expert and the K weighted rows in k order
 *                     and stores the slice into every rank's output, fence, flag
 *   wait              the pass is complete on a rank when it has every rank's slice flag
 *
 * The pass number lives in device memory and the pass reads nothing on the host, so
 * b200_ep_forward records it into a CUDA graph on its third call with the same (x, T) and
 * replays it afterwards.
 *
 * Every wait is bounded (spin limit); when one runs out the kernel sets the library's
 * status word and returns, and the next b200_stream_status() reports B200_ECUDA.  The
 * exchange uses plain peer stores only (no TMA, no multicast).
 */
#ifndef B200EP_H
#define B200EP_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct b200_ep b200_ep;

#define B200_EP_HANDLE_BYTES 64      /* a rank's exported block handle (cudaIpcMemHandle_t) */
#define B200_EP_MAX_WORLD 16

/* max_tokens: the largest T a forward pass will be given.  capacity_rows: rows one rank
 * may send to one other rank in one pass (0: the worst case, every slot of its slice);
 * a pass that would exceed it sets the status word and delivers the first capacity_rows. */
int b200_ep_create(b200_ep** out, int rank, int world, int d, int E, int ne, int K, int SH, int qkind, int max_tokens,
                   int capacity_rows);
int b200_ep_destroy(b200_ep* ep);
/* Device pointers, kept by reference: router [ne, d] fp32 and its bias [ne] (or NULL),
 * replicated; this rank's experts gates / ups [ne / world * E, d], downs [ne / world * d, E]
 * in the storage form of qkind; the replicated shared expert (or NULLs). */
int b200_ep_set_weights(b200_ep* ep, const float* router_w, const float* router_bias, const void* gates_local,
                        const void* ups_local, const void* downs_local, const void* sh_gate, const void* sh_up,
                        const void* sh_down);
/* Across processes: each rank exports its block, the B200_EP_HANDLE_BYTES travel by whatever
 * the application has (the reference passes its NCCL id through a file, GAI_NCCL_ID_FILE),
 * and every rank connects with all ranks' handles in rank order. */
int b200_ep_export(b200_ep* ep, void* handle_out);
int b200_ep_connect(b200_ep* ep, const void* handles_all);
/* The same through files <dir>/b200ep.<rank> (written atomically, polled up to timeout_ms). */
int b200_ep_rendezvous_dir(b200_ep* ep, const char* dir, int timeout_ms);
/* Ranks living in this process (tests, several GPUs under one process): peers[world]. */
int b200_ep_connect_local(b200_ep* ep, b200_ep* const* peers);

/* The whole layer: x [T, d] fp32 device (replicated), result in b200_ep_output.  Enqueues on
 * the library's stream and returns; ranks must call it the same number of times with the
 * same T. */
int b200_ep_forward(b200_ep* ep, const float* x, int T);
/* The same in its four stream-ordered phases (0 route + dispatch, 1 experts + return,
 * 2 combine + gather, 3 wait for all slices), always eager.  Ranks that share one GPU must run phase p for
 * every rank before phase p + 1 of any (their waits then never spin). */
int b200_ep_phase(b200_ep* ep, int phase, const float* x, int T);
/* out_dev: [T, d] fp32 of the last pass (valid until the next pass begins on any rank). */
int b200_ep_output(b200_ep* ep, const float** out_dev);
/* Routing of this rank's slice in the last pass: idx [n, K] int32, w [n, K] fp32 (device),
 * n = slice length. */
int b200_ep_routing(b200_ep* ep, const int32_t** idx_dev, const float** w_dev, int* n_slice);
/* Test hook: iterations a flag wait may spin (0 restores the default). */
int b200_ep_set_spin_limit(b200_ep* ep, int spin_limit);
/* Bytes the last pass moved over the links from this rank: the fp16 rows of slots whose expert
 * lives elsewhere, as many fp32 result rows, and the output slice to world - 1 peers; counted on
 * the host from the pass's expert offsets (synchronises). */
int b200_ep_link_bytes(b200_ep* ep, double* bytes);

#ifdef __cplusplus
}
#endif
#endif /* B200EP_H */
