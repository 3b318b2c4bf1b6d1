/*
 * moe_b200.h — C ABI of libmoe_b200.so: the MoE routing / dispatch hot path
 * of santiweide/moe-routers rebuilt for NVIDIA B200 (sm_100a).
 *
 * Conventions
 *   - every entry point returns an int status (MOE_OK == 0); nothing calls
 *     exit(), nothing throws;
 *   - all pointers are DEVICE pointers unless the name ends in _host;
 *   - no entry point allocates or frees device memory and none synchronises
 *     the host (the one exception says so); scratch comes from a caller-owned
 *     workspace sized by moe_workspace_bytes();
 *   - `stream` is a cudaStream_t passed as void*; work is enqueued on it;
 *   - element type codes: MOE_F16, MOE_BF16, MOE_F32;
 *   - the library keeps no mutable global state: calls on different streams
 *     with different workspaces are independent (moe_pack_static, which owns
 *     its scratch, says what it shares);
 *   - environment switches, read once per process, all default to the fast
 *     path: MOE_B200_PDL=0 (no programmatic dependent launch between the
 *     route kernels; moe_set_pdl changes it at run time); grouped GEMM
 *     variants, also changed at run time by moe_set_gemm_mode: MOE_B200_CTA2=0
 *     (no two-CTA kernel), MOE_B200_CTA2_ISSUERS=1 (one MMA-issuing thread
 *     in it), MOE_B200_PAIR=0 (single-tile work units), MOE_B200_M64=0
 *     (128-row tiles only), MOE_B200_GEMM_PRODUCERS=1 (one TMA-issuing
 *     warp); MOE_B200_ROUTER_BULK=0 (router kernel: split-K partials exchanged
 *     with remote stores also where a bulk copy would do),
 *     MOE_B200_ROUTER_PREFETCH=0 (no L2 prefetch of the tokens ahead of the
 *     dependency wait);
 *     MOE_B200_SINKHORN_CLUSTER=8 (portable cluster size).
 *
 * Each declaration names the piece of the reference (path:lines inside
 * santiweide/moe-routers) that it replaces.
 */
#ifndef MOE_B200_H_
#define MOE_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum {
  MOE_OK = 0,
  MOE_ERR_ARG = 1,        /* bad argument (null pointer, size, dtype, alignment) */
  MOE_ERR_UNSUPPORTED = 2,/* shape outside what the kernels are built for */
  MOE_ERR_WORKSPACE = 3,  /* workspace missing or too small */
  MOE_ERR_LAUNCH = 4,     /* CUDA reported a launch / driver error */
  MOE_ERR_DEVICE = 5      /* a kernel recorded an error in the status block */
};

enum { MOE_F16 = 0, MOE_BF16 = 1, MOE_F32 = 2 };

/* Activation fused into the grouped GEMM epilogue. */
enum { MOE_ACT_NONE = 0, MOE_ACT_GELU = 1, MOE_ACT_SILU = 2, MOE_ACT_SWIGLU = 3 };

/* Storage of a weight matrix: MOE_W_KN = [K,N] row-major (N contiguous, what
 * grouped_ffn_forward is given), MOE_W_NK = [N,K] row-major (nn.Linear). */
enum { MOE_W_KN = 0, MOE_W_NK = 1 };

/* Library version and a human-readable text for the last non-OK status
 * returned on the calling thread. */
int moe_version(void);
const char* moe_last_error(void);

/* Bytes of workspace the routing entry points need for `tokens` tokens,
 * `experts` experts and `top_k` picks.  The first 256 bytes are the status
 * block (see moe_read_status). */
size_t moe_workspace_bytes(int tokens, int experts, int top_k);

/* Zero the status block of a workspace (async on `stream`).  Call once after
 * allocating the workspace. */
int moe_workspace_init(void* workspace, size_t workspace_bytes, void* stream);

/* Limit, in nanoseconds, of every bounded device-side wait of kernels that are given this workspace
 * (mbarrier waits, grid barriers, moe_ep_wait); 0 restores the default of 2 s.  Stored in the status
 * block by an async copy on `stream`; call it outside stream capture.  A wait that runs out records
 * a code in the status block (see moe_read_status) and the kernel returns; nothing traps.
 * (Setup helper; the reference has no counterpart: its kernels never wait.) */
int moe_set_wait_limit(void* workspace, size_t workspace_bytes, unsigned long long limit_ns, void* stream);

/* Kernel launches this library has issued in this process so far (all threads, captured launches
 * count when they are captured).  Measurement helper; no counterpart in the reference. */
long long moe_launch_count(void);

/* Programmatic dependent launch between the kernels of a route (the scatter may start its input
 * prefetch under the router kernel's epilogue): 0 = plain stream order, non-zero = on (default,
 * unless MOE_B200_PDL=0 is in the environment).  Process-wide; takes effect for launches issued
 * after the call.  Measurement helper; no counterpart in the reference. */
int moe_set_pdl(int enabled);

/* Variants the grouped GEMM may use; every combination computes the same result bits, the default
 * (all on) is the fastest measured.  moe_set_gemm_mode(mode) replaces the set for launches issued
 * after the call (process-wide) and returns the previous one; a negative mode only reads it.
 * Measurement and test helper; no counterpart in the reference. */
enum {
  MOE_GEMM_TWO_CTA = 1,       /* two-CTA kernel (tcgen05 cta_group::2) for experts with >= 512 rows on average */
  MOE_GEMM_TWO_ISSUERS = 2,   /* two MMA-issuing threads in the two-CTA kernel */
  MOE_GEMM_TILE_PAIRS = 4,    /* one-CTA kernel: two 128-row tiles per work unit for such experts */
  MOE_GEMM_M64 = 8,           /* one-CTA kernel: a last tile of <= 64 rows as UMMA M=64 */
  MOE_GEMM_TWO_PRODUCERS = 16,/* one-CTA kernel: second TMA-issuing warp for single-tile units */
  MOE_GEMM_ALL = 31
};
int moe_set_gemm_mode(int mode);

/* Copy the status block's first word to the host.  THIS CALL SYNCHRONISES
 * `stream`.  0 means no kernel recorded an error; otherwise the value encodes
 * which bounded wait gave up (see moe_last_error). */
int moe_read_status(const void* workspace, void* stream, int* status_host);

/*
 * Top-k selection with softmax gates over the selected logits.
 * Replaces: fused_select_cuda.forward(logits, k) as called by CUDATopKRouter
 * (models/decoder_moe.py:137-151), torch.topk + softmax of TorchTopKRouter
 * (models/decoder_moe.py:58-62) and top2_select_64_kernel
 * (kernels/fused_select.cu:47-113).
 *   logits [tokens, experts] row-major, dtype code `logits_dtype`
 *   idx    [tokens, top_k] int32, descending logit order, lowest index wins ties
 *   gates  [tokens, top_k] float32, softmax over the selected values
 * Limits: 1 <= top_k <= 8, top_k <= experts <= 1024.
 */
int moe_topk_select(const void* logits, int logits_dtype, int tokens, int experts, int top_k,
                    int32_t* idx, float* gates, void* stream);

/*
 * Count, scan and pack: expert-contiguous copy of the raw token rows.
 * Replaces: count_expert_kernel, the CUB scan, the host read-back and
 * pack_copy_kernel (kernels/fused_select.cu:116-198, :256-308) and the torch
 * pack _pack_routes (bench_router.py:57-78).
 *   x         [tokens, d] row-major, `elem_bytes` bytes per element (2 or 4)
 *   idx       [tokens, top_k] int32 expert ids in [0, experts)
 *   counts    [experts] int32            routes per expert
 *   offsets   [experts + 1] int32        exclusive prefix, offsets[experts] = tokens*top_k
 *   packed    [tokens*top_k, d]          row p holds x[row_route[p] / top_k], bit for bit
 *   row_route [tokens*top_k] int32       route id (t*top_k + j) stored in packed row p
 *   route_row [tokens*top_k] int32       inverse permutation (may be NULL)
 * Order inside an expert segment is ascending route id (deterministic).
 * `packed` may be NULL to compute only counts / offsets / maps.
 */
int moe_pack(const void* x, int elem_bytes, const int32_t* idx, int tokens, int d, int experts,
             int top_k, int32_t* counts, int32_t* offsets, void* packed, int32_t* row_route,
             int32_t* route_row, void* workspace, size_t workspace_bytes, void* stream);

/*
 * Select + count + scan + pack from given logits: the reference's whole operator
 * fused_select_forward(logits, x) (kernels/fused_select.cu:203-311: five kernels, two memsets,
 * six allocations and one host round trip) as two launches: the select kernel also writes the
 * per-tile expert histograms, the scatter derives offsets from them.  Arguments as in
 * moe_topk_select and moe_pack; any experts <= 1024 and top_k <= 8.
 */
int moe_fused_select(const void* logits, int logits_dtype, const void* x, int elem_bytes, int tokens, int d,
                     int experts, int top_k, int32_t* idx, float* gates, int32_t* counts, int32_t* offsets,
                     void* packed, int32_t* row_route, int32_t* route_row, void* workspace,
                     size_t workspace_bytes, void* stream);

/*
 * The scatter half of the pack on its own (offsets, ranks and row copies), reading the per-tile
 * histograms that a preceding moe_router_gemm_select / moe_route_fused / moe_fused_select call with
 * the same workspace, token count and expert count left in the workspace.  It is what
 * moe_route_fused launches second; exposed so that the stage can be driven and timed by itself
 * (T_pack of bench_router.py:547-552).  Arguments as in moe_pack.
 */
int moe_pack_scatter(const void* x, int elem_bytes, const int32_t* idx, int tokens, int d, int experts,
                     int top_k, int32_t* counts, int32_t* offsets, void* packed, int32_t* row_route,
                     int32_t* route_row, void* workspace, size_t workspace_bytes, void* stream);

/*
 * moe_pack_scatter with one destination segment per expert: the rows routed to expert e are stored in
 * canonical order from seg_base[e] on (device array of `experts` 16-byte aligned addresses, which
 * may lie in peers' memory) instead of at packed[offsets[e]]; counts, offsets and the maps are
 * written as by moe_pack.  Rows must be a multiple of 16 bytes.  With the table of
 * moe_ep_segment_bases this is the dispatch of the expert-parallel layer: the pack writes every row
 * straight into the owner's inbox over NVLink (bulk stores), replacing pack + all_to_all_single
 * (bench_2gpu_pcie.py:305-372, :466-494).
 */
int moe_pack_scatter_to(const void* x, int elem_bytes, const int32_t* idx, int tokens, int d, int experts,
                        int top_k, int32_t* counts, int32_t* offsets, void* const* seg_base, int32_t* row_route,
                        int32_t* route_row, void* workspace, size_t workspace_bytes, void* stream);

/*
 * moe_pack for callers that cannot allocate.  (No counterpart in the reference.)
 * Same inputs, outputs and ordering as moe_pack, but the scratch that moe_pack takes from a
 * caller-owned workspace comes from a 256 KiB array built into the library image, so the call
 * needs no cudaMalloc on anybody's side: meant for code that runs inside a fixed memory plan or
 * inside a host hook where device allocation is forbidden or may stall the device.
 *   - limits: tokens <= 8192 and experts <= 256; larger sizes return MOE_ERR_UNSUPPORTED
 *     (use moe_pack);
 *   - the call allocates and frees nothing, and calls no allocating library routine;
 *   - the first call on each device looks up the array's device address (once, cached); make
 *     that first call before any stream capture begins on that device;
 *   - all calls on a device share the one array: two calls whose kernels may overlap on the GPU
 *     (different streams without ordering between them) race; serialise them.  The array keeps
 *     the last call's contents, and every word a call reads it has written first;
 *   - device_status: NULL, or one int32 on the device that receives a non-zero code if an expert
 *     index is out of range (the caller clears it).
 */
int moe_pack_static(const void* x, int elem_bytes, const int32_t* idx, int tokens, int d, int experts,
                    int top_k, int32_t* counts, int32_t* offsets, void* packed, int32_t* row_route,
                    int32_t* route_row, int32_t* device_status, void* stream);

/*
 * Gate-weighted un-permute and sum over the top_k picks:
 *   out[t] = sum_j gates[t,j] * y[route_row[t*top_k + j]]   (fp32 accumulate)
 * Replaces: `expert(x_e) * w_e` + index_add_ (models/decoder_moe.py:270-271).
 *   y [tokens*top_k, d] and out [tokens, d] have dtype `dtype` (MOE_F16 / MOE_BF16).
 */
int moe_combine(const void* y, int dtype, const float* gates, const int32_t* route_row, int tokens,
                int d, int top_k, void* out, void* stream);

/*
 * Fused route: router logit GEMM (tcgen05 / TMEM, TMA-fed) whose epilogue adds
 * the skew bias, selects top-k and computes the gates, followed by the pack.
 * Replaces the whole `fused_select` strategy: x @ w.t() + skew
 * (bench_router.py:512-516) and fused_select_forward
 * (kernels/fused_select.cu:203-311); the logits never go to HBM unless
 * `logits_out` is given.
 *   x [tokens, d], w_router [experts, d]: both `dtype` (MOE_F16 or MOE_BF16), row-major, d % 8 == 0
 *   skew: logits[:, :skew_experts] += skew_bias, applied after the logits are
 *         rounded to `dtype` (the dtype the reference computes them in)
 *   logits_out: NULL or [tokens, experts] float32 receiving the values the
 *         selection saw
 *   remaining outputs as in moe_topk_select and moe_pack.
 * Limits: experts <= 256, 1 <= top_k <= 8, top_k <= experts, d % 8 == 0.
 */
int moe_route_fused(const void* x, const void* w_router, int dtype, int tokens, int d, int experts, int top_k,
                    int skew_experts, float skew_bias, int32_t* idx, float* gates, int32_t* counts,
                    int32_t* offsets, void* packed, int32_t* row_route, int32_t* route_row,
                    float* logits_out, void* workspace, size_t workspace_bytes, void* stream);

/* The logit GEMM + select half of moe_route_fused on its own (T_logit +
 * T_select of bench_router.py:512-545 in one launch). */
int moe_router_gemm_select(const void* x, const void* w_router, int dtype, int tokens, int d, int experts,
                           int top_k, int skew_experts, float skew_bias, int32_t* idx, float* gates,
                           float* logits_out, void* workspace, size_t workspace_bytes, void* stream);

/*
 * Sinkhorn-balanced routing.
 * Replaces: SinkhornRouter.forward (models/decoder_moe.py:92-123) and the
 * unbuilt kernels of kernels/fused_sinkhorn.cu:56-209.
 *   q = exp(logits/temperature - rowmax); iters x { rows /= (sum+eps);
 *   cols = cols/(sum+eps) * tokens/experts }; rows /= (sum+eps); top-k of q,
 *   gates = vals / (sum(vals) + eps).
 *   idx [tokens, top_k] int32, gates [tokens, top_k] float32.
 * Limits: top_k <= 8, experts <= 1024, tokens * experts * 4 bytes / (number of SMs) must fit in
 * shared memory (about 7 M matrix entries on a B200).  The kernel runs as a cooperative grid
 * with one grid barrier per iteration; if a barrier wait gives up, the status block records it
 * and the workspace must be re-initialised with moe_workspace_init.
 */
int moe_sinkhorn(const void* logits, int logits_dtype, int tokens, int experts, int top_k, int iters,
                 float epsilon, float temperature, int32_t* idx, float* gates, void* workspace,
                 size_t workspace_bytes, void* stream);

/*
 * Grouped expert GEMM over expert-contiguous rows (tcgen05 / TMEM, TMA-fed,
 * persistent tile scheduler driven by the device-side offsets):
 *   for every expert e: C[offsets[e]:offsets[e+1], :] =
 *         act( A[offsets[e]:offsets[e+1], :] @ W[e] ) (* row_scale[row])
 * Replaces: grouped_ffn_forward (kernels/grouped_ffn.cu:53-136) and the
 * per-expert loops (bench_2gpu_pcie.py:123-171, models/decoder_moe.py:256-273,
 * fused_select.py:74-93).
 *   a [rows, K] row-major; w: `experts` matrices, stride_w elements apart,
 *   each [K,N] (MOE_W_KN) or [N,K] (MOE_W_NK); c [rows, N]; all 16-bit (`dtype`)
 *   (for MOE_ACT_SWIGLU the weight has 2N output features, gate then up, and
 *   c = silu(gate) * up has N columns)
 *   offsets [experts+1] int32 on the device; `rows` is the capacity of a / c
 *   row_scale: NULL or float32 [rows] multiplied into the result rows.
 *   bias:      NULL or [experts, output features of W] in `dtype`, added before the activation
 *              (the `+ b1[e]` / `+ b2[e]` loops of fused_select.py:74-93).
 *   dtype:     MOE_F16 or MOE_BF16 for a, w, bias and c.
 *   sm_margin: SMs the persistent grid leaves free (0 = use all), so that a communication
 *              kernel running on another stream can make progress next to it.
 * Limits: K % 8 == 0; N % 16 == 0 for [N,K] weights, N % 64 == 0 for [K,N] weights;
 * experts <= 1024.
 */
int moe_grouped_gemm(const void* a, const void* w, void* c, const int32_t* offsets, int experts,
                     int rows, int K, int N, int w_layout, int64_t stride_w, int activation,
                     const float* row_scale, const void* bias, int dtype, int sm_margin, void* workspace,
                     size_t workspace_bytes, void* stream);

/*
 * moe_grouped_gemm with scattered output rows: row r of the result is stored at c_rows[r] (a device
 * array of `rows` addresses, each 16-byte aligned with room for N elements) instead of row r of a
 * dense C.  The addresses may point into another GPU's memory mapped into this process
 * (moe_ipc_open): the expert-parallel layer passes the table built by moe_ep_row_targets so that the
 * second expert GEMM returns every result row to the packed slot of the rank it came from, from
 * inside the GEMM kernel (128-byte row pieces, plain stores).
 * Replaces, together with moe_ep_row_targets: the per-expert MLP loop followed by a separate return
 * exchange, which the reference leaves out (bench_2gpu_pcie.py:123-171, :20-25).  All other
 * arguments as moe_grouped_gemm.
 */
int moe_grouped_gemm_rows(const void* a, const void* w, void* const* c_rows, const int32_t* offsets, int experts,
                          int rows, int K, int N, int w_layout, int64_t stride_w, int activation,
                          const float* row_scale, const void* bias, int dtype, int sm_margin, void* workspace,
                          size_t workspace_bytes, void* stream);

/*
 * Expert-parallel re-bucketing of rows received by the dispatch all-to-all.
 * Replaces: the argsort / index_select / bincount bucketing of received rows
 * (bench_2gpu_pcie.py:130-171) on the owner rank.
 *   counts_all [world, experts] int32: the all-gathered per-rank route counts
 *   src / dst  [rows, d]: forward (backward == 0) moves source-major rows
 *              ([source rank][local expert][rows], what the all-to-all delivers) to expert-major
 *              order ([local expert][source rank][rows], what moe_grouped_gemm reads) and writes
 *              local_offsets int32 [experts/world + 1]; backward != 0 is the inverse move and
 *              ignores local_offsets (may be NULL)
 *   skip_src:  a source rank whose rows are not in the buffers (-1 for none): the rank itself,
 *              when its own rows bypass the all-to-all (bench_2gpu_pcie.py:23-25)
 *   first_local_expert, num_local_experts: the range of this rank's experts the buffers hold (the
 *              layer exchanges and computes the local experts in chunks so that the exchange of one
 *              chunk overlaps the FFN of another); local_offsets then has num_local_experts + 1 entries
 */
int moe_ep_rebucket(const void* src, void* dst, const int32_t* counts_all, int experts, int world, int rank,
                    int skip_src, int backward, int d, int elem_bytes, int first_local_expert,
                    int num_local_experts, int32_t* local_offsets, void* stream);

/*
 * Device-initiated dispatch (combine == 0) and combine (combine != 0) over peer memory.
 * Replaces: the all_to_all_single exchanges of rows and expert ids plus the receiver-side
 * bucketing (bench_2gpu_pcie.py:460-488, :130-171).
 *   peer_bufs: DEVICE array of `world` pointers; entry p is rank p's inbox (dispatch) or rank p's
 *              packed-order result buffer (combine), mapped into this process (CUDA IPC); the
 *              entry for the rank itself is its own buffer.  All must be 16-byte aligned.
 *   dispatch:  local = this rank's packed rows; every expert segment is stored into its owner's
 *              inbox at its expert-major position, so the owner's rows arrive already grouped by
 *              expert; local_offsets (int32 [experts/world + 1]) receives this rank's own inbox
 *              offsets for moe_grouped_gemm.
 *   combine:   local = this rank's expert-major FFN output; every segment is stored into the packed
 *              slot of the rank it came from.
 * The kernel only stores; the caller orders the phases across ranks (every rank must have finished
 * its dispatch before any rank reads its inbox, and likewise for the combine).
 */
/* Let kernels on the current device store into memory of `peer_device` (cudaDeviceEnablePeerAccess;
 * already enabled is not an error).  Call once per peer before the first moe_ep_push.
 * (Setup helper; the reference has no counterpart.) */
int moe_enable_peer_access(int peer_device);

/* Map / unmap a peer process's device allocation (64-byte CUDA IPC handle of its base) for access
 * from the current device.  Setup helpers; the reference has no counterpart. */
int moe_ipc_open(const void* handle64, void** base_out);
int moe_ipc_close(void* base);
/* Export side: the 64-byte IPC handle of the device allocation that contains `ptr` (host buffer
 * handle64_out) and the byte offset of `ptr` inside that allocation; the peer maps the handle with
 * moe_ipc_open and adds the offset.  The allocation must come from cudaMalloc. */
int moe_ipc_export(const void* ptr, void* handle64_out, size_t* offset_out);

/* PCI address of CUDA device `device` as "domain:bus:device.function" (cudaDeviceGetPCIBusId) into
 * the host buffer `out` of `len` bytes (>= 16).  Host-side helper: HostRouter uses it to place its
 * pinned staging buffers on the NUMA node the GPU is attached to.  No counterpart in the reference. */
int moe_device_pci_bus_id(int device, char* out, int len);

int moe_ep_push(const void* local, void* const* peer_bufs, const int32_t* counts_all, int experts, int world,
                int rank, int combine, int d, int elem_bytes, int32_t* local_offsets, void* stream);

/*
 * Rank-to-rank signals over peer mappings: the phase ordering of the expert-parallel layer without
 * a collective.  Replaces: the all_to_all_single of the split sizes with its `.tolist()` host read and
 * the implicit ordering of the blocking collectives (bench_2gpu_pcie.py:460-494).
 *   Every rank owns a flag table int32 [slots][world], zero at start, in memory the peers have mapped.
 *   moe_ep_signal: first copies `payload` (NULL, or `payload_words` int32 on this device, e.g. the
 *     per-expert counts) to peer_payload[p] + payload_offset_words for every rank p, then makes all
 *     earlier stores of this rank visible system-wide and stores `value` into entry [slot][rank] of
 *     every rank's table (peer_flags: DEVICE array of `world` table addresses; own entry = own table).
 *   moe_ep_wait: polls this rank's OWN table until every entry of `slot` has reached `value`
 *     (signed distance, so the counter may wrap).  Bounded by the workspace's wait limit
 *     (moe_set_wait_limit, default 2 s): on expiry the status block gets code 0x400 | rank-that-never-
 *     signalled and the kernel returns.
 *   Values must grow from call to call (pass a call counter); tables are never cleared.
 *   One process per GPU: a waiting kernel and the kernels that signal it must run on different GPUs
 *   (or the signals must already be in memory); two such kernels on one GPU may never overlap.
 */
int moe_ep_signal(void* const* peer_flags, int world, int rank, int slot, int value, const int32_t* payload,
                  void* const* peer_payload, size_t payload_offset_words, int payload_words, void* stream);
int moe_ep_wait(const int32_t* flags, int world, int slot, int value, void* workspace, size_t workspace_bytes,
                void* stream);
/* moe_ep_signal followed by moe_ep_wait on the same slot and value, as ONE kernel launch (what the
 * layer uses between its phases).  Only where every rank runs on its own GPU: with several ranks
 * emulated on one GPU the wait would be for signals of launches queued behind it. */
int moe_ep_sync(void* const* peer_flags, const int32_t* flags, int world, int rank, int slot, int value,
                const int32_t* payload, void* const* peer_payload, size_t payload_offset_words, int payload_words,
                void* workspace, size_t workspace_bytes, void* stream);

/*
 * Dispatch destinations: seg_base[g] (g = global expert) = address, inside inbox_bufs[owner of g]
 * (device array of `world` inbox base addresses, peers' through their mappings), of the first row
 * this rank contributes to expert g in the owner's expert-major inbox; also writes this rank's own
 * local_offsets int32 [experts/world + 1] (may be NULL).  Input of moe_pack_scatter_to.
 * Replaces: the send-split bookkeeping of route_and_pack (bench_2gpu_pcie.py:305-372).
 */
int moe_ep_segment_bases(void* const* inbox_bufs, const int32_t* counts_all, int experts, int world, int rank,
                         int d, int elem_bytes, void** seg_base, int32_t* local_offsets, void* stream);

/*
 * Return addresses for the combine direction: row_ptrs[i] (i over this rank's expert-major inbox rows,
 * the order moe_ep_push dispatch produces) = address of the packed slot that row came from, inside
 * home_bufs[source rank] (device array of `world` base addresses of the ranks' [k*T, d] result
 * buffers, peers' through their mappings).  Input of moe_grouped_gemm_rows.
 * Replaces: the bookkeeping of the (missing) return exchange, bench_2gpu_pcie.py:20-25.
 */
int moe_ep_row_targets(void* const* home_bufs, const int32_t* counts_all, int experts, int world, int rank,
                       int d, int elem_bytes, void** row_ptrs, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* MOE_B200_H_ */
