/*
 * C ABI of the B200 (sm_100a) weight-only quantised GEMM backend.
 *
 * Plain pointers and sizes only; every pointer is a DEVICE pointer on the current
 * CUDA device unless stated otherwise.  Calls enqueue work on `cuda_stream`
 * (a cudaStream_t passed as void*) and do not synchronise, allocate or free
 * device memory, so they can be recorded into a CUDA graph.  Every function
 * returns DXB_OK (0) or a negative DXB_ERR_* code; nothing throws.
 *
 * The entry points are what a host binding for the reference's kernel slot
 *     impl(x, qweight, scales, zeros, bias, group_size) -> Tensor
 * needs (python/dexter/ops/reference/gemm.py:82-89 and
 * python/dexter/ops/gfx1151/gemm/quantized.py:223-263 in the reference).
 *
 * Tensor layouts are the reference quantiser's (python/dexter/quant.py:34-133):
 *   x        [M, K]    bf16, row stride `ldx` elements (>= K)
 *   qweight  int4: [K/2, N] uint8, byte [i, n] = row i (low nibble) and row
 *            i + K/2 (high nibble); int8: [K, N] uint8.  Row stride N.
 *   scales   [K/group_size, N] bf16
 *   zeros    [K/group_size, N] bf16 or NULL (symmetric: zero point 2^(bits-1));
 *            4-bit zero points are stored with +128 added (quant.py:118-122)
 *   bias     [N] bf16 or NULL
 *   out      [M, N]    bf16, row stride `ldo` elements (>= N)
 */
#ifndef DEXTER_B200_H_
#define DEXTER_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum {
  DXB_OK = 0,
  DXB_ERR_BITS = -1,           /* bits not 4 or 8  (ValueError in ops/__init__.py:110-111) */
  DXB_ERR_NULL = -2,           /* a required pointer is NULL */
  DXB_ERR_SHAPE = -3,          /* K vs group / packing / stride mismatch (quantized.py:225-226) */
  DXB_ERR_UNSUPPORTED = -4,    /* shape outside what this build can run (quantized.py:220) */
  DXB_ERR_WORKSPACE = -5,      /* workspace NULL or smaller than dxb_workspace_bytes() */
  DXB_ERR_TENSORMAP = -6,      /* cuTensorMapEncodeTiled refused the tensor */
  DXB_ERR_CUDA = -7,           /* launch failed; see cudaGetLastError */
  DXB_ERR_KERNEL_TIMEOUT = -8, /* a bounded in-kernel wait ran out (read via dxb_read_status) */
  DXB_ERR_SCRATCH_LIMIT = -9   /* dxb_wq_gemm_static: needs more than the built-in 24 MiB */
};

/*
 * out = x @ dequant(qweight, scales, zeros) (+ bias).
 * Replaces the reference's _launch() + Triton kernel for `bits` = 4 or 8
 * (python/dexter/ops/gfx1151/gemm/quantized.py:47-183, 223-249).
 * `workspace` holds a status word, tile counters and split-K partial sums; it
 * must be at least dxb_workspace_bytes() and zero-filled once before its first
 * use (the kernel leaves it clean after every normal completion).  Two calls
 * that may overlap on the GPU need different workspaces.
 * `max_ctas` <= 0 lets the library use every SM; a positive value caps the grid, so
 * that several independent GEMMs can run side by side on different streams.
 * Any M: up to 128 tokens are one accumulator block; more tokens are processed as blocks of
 * 128 inside ONE launch (every (token block, 128-column tile) pair is a tile of the grid).
 */
int dxb_wq_gemm(int bits, const void* x, int64_t ldx, const void* qweight, const void* scales,
                const void* zeros, const void* bias, void* out, int64_t ldo, int M, int N, int K,
                int group_size, void* workspace, size_t workspace_bytes, int max_ctas,
                void* cuda_stream);

/* The registered kernels gemm/w4a16 and gemm/w8a16
 * (python/dexter/ops/gfx1151/gemm/quantized.py:252-263). */
int dxb_w4a16(const void* x, int64_t ldx, const void* qweight, const void* scales,
              const void* zeros, const void* bias, void* out, int64_t ldo, int M, int N, int K,
              int group_size, void* workspace, size_t workspace_bytes, void* cuda_stream);
int dxb_w8a16(const void* x, int64_t ldx, const void* qweight, const void* scales,
              const void* zeros, const void* bias, void* out, int64_t ldo, int M, int N, int K,
              int group_size, void* workspace, size_t workspace_bytes, void* cuda_stream);

/*
 * Same GEMM as dxb_wq_gemm for callers that cannot hand over a workspace because
 * they are not allowed to allocate device memory at all: code running inside
 * another framework's memory plan (a serving runtime that has already carved up
 * the whole GPU, a plugin whose host forbids cudaMalloc on its threads), or code
 * that must stay free of allocator calls because those may synchronise or fail
 * at a bad moment.  This entry point has no counterpart in the reference; it is
 * an addition of this library.
 *
 * The split-K scratch (status word, tile counters, fp32 partial sums) is a fixed
 * 24 MiB array inside the library image; each GPU that loads the library holds it
 * until the process exits.  The call itself calls no cudaMalloc / cudaFree and no
 * allocating library routine.  Limits and rules:
 *   - a problem whose scratch need (dxb_workspace_bytes) exceeds 24 MiB is refused
 *     with DXB_ERR_SCRATCH_LIMIT and nothing is launched (the shapes of the 5B and
 *     14B backbones at up to 128 tokens per launch fit);
 *   - the first call on each device looks up the array's device address; make that
 *     first call outside any stream capture;
 *   - all calls share the one array: the counters and the status word are cleared
 *     (cudaMemsetAsync on `cuda_stream`) at the start of every call, partial sums
 *     are overwritten before use; two calls that may run on the GPU at the same
 *     time (different streams, no ordering) race on it and must not be made.
 */
int dxb_wq_gemm_static(int bits, const void* x, int64_t ldx, const void* qweight,
                       const void* scales, const void* zeros, const void* bias, void* out,
                       int64_t ldo, int M, int N, int K, int group_size, void* cuda_stream);

/*
 * Several GEMMs of one layer in ONE launch.  The reference runs a block's linears as
 * successive calls of the kernel slot, one launch each (ops.linear,
 * python/dexter/ops/__init__.py:89-112, called per projection from
 * python/dexter/models/layers.py:44-50); at
 * M <= 128 tokens each of those launches is dominated by its start-up and drain.  A
 * chain hands the whole list to one persistent grid (one CTA per SM): every CTA works
 * through the items in order, the packed-weight pipeline of item i+1 fills while item
 * i drains, and an item whose activations are an earlier item's output waits on a
 * completion count in global memory instead of a kernel boundary.
 *
 * Rules:
 *   - 1 <= n_items <= DXB_CHAIN_MAX; every item must be a shape the tensor-core kernel
 *     takes (dxb_uses_tensor_cores, M <= 128, 16-byte aligned pointers and strides) with
 *     at least 8 units of 128 (int4) or 64 (int8) rows of K; all items share `bits` and
 *     either all or none have zero points; otherwise DXB_ERR_UNSUPPORTED and nothing is
 *     launched (call dxb_wq_gemm per item instead).
 *   - depends_on = index of the EARLIER item whose `out` buffer this item's `x` reads,
 *     or -1 when `x` is ready before the call.  An item may depend on one item only.
 *     Items are started in list order; placing an independent item between a producer
 *     and its consumer hides the hand-over completely.
 *   - no `out` buffer may overlap another item's `out` or any item's `x` other than
 *     that of the items that name it in depends_on.
 *   - `workspace`: at least dxb_chain_workspace_bytes() (a status word and completion
 *     counts; partial sums stay in shared memory), 256-byte aligned, zero-filled once
 *     before its first use; the kernel leaves it clean after every normal completion.
 *     Calls that may overlap on the GPU need different workspaces.
 *   - the grid (clusters of 2, 4 or 8 CTAs, as many as are resident at once) is sized for
 *     a GPU that this stream has to itself while the chain runs.  Every in-kernel wait is
 *     bounded: if part of the grid cannot become resident because other work holds SMs,
 *     the call ends with DXB_ERR_KERNEL_TIMEOUT in dxb_read_status(workspace), it does
 *     not hang.
 * Each item computes what dxb_wq_gemm computes for it (same dequantisation, fp32
 * accumulation, bf16 rounding, bias order); only the split of the K range differs, and the
 * partial sums of a tile are always added in the same order, so runs are reproducible.
 */
#define DXB_CHAIN_MAX 32
typedef struct dxb_chain_item {
  const void* x;
  int64_t ldx;
  const void* qweight;
  const void* scales;
  const void* zeros;
  const void* bias;
  void* out;
  int64_t ldo;
  int M, N, K, group_size;
  int depends_on;
} dxb_chain_item;

size_t dxb_chain_workspace_bytes(int bits, const dxb_chain_item* items, int n_items, int max_ctas);
int dxb_wq_gemm_chain(int bits, const dxb_chain_item* items, int n_items, void* workspace,
                      size_t workspace_bytes, int max_ctas, void* cuda_stream);

/*
 * Tensor-parallel glue for the few-token regime: sum of the row-parallel linears' partial
 * outputs over the ranks of one NVLink domain, every rank receiving the full sum.  The
 * reference has no tensor parallelism, so this replaces nothing there; it stands where a
 * library all-reduce would, which at 83 x 3072 bf16 (0.5 MB) is mostly latency.
 *
 * peer_regions[r] = rank r's region of peer-mapped memory AS MAPPED IN THIS PROCESS (host
 * array of `world` device pointers, 16-byte aligned), each dxb_peer_allreduce_bytes(world,
 * capacity_elems) bytes, zero-filled on every rank before anyone's first call and used for
 * nothing else.  `partial` and `out` are ordinary local buffers of `elems` bf16 (elems a
 * multiple of 8, <= capacity_elems).  All ranks must make the same sequence of calls with
 * the same `elems`; each rank runs on its own GPU.  One kernel per call: plain 16-byte
 * stores into the peers' regions, system-scope release/acquire flags, a bounded wait (about
 * a second, then DXB_ERR_KERNEL_TIMEOUT in *status, a local int, may be NULL), the sum in
 * fp32 in rank order (identical bits on every rank), one rounding to bf16.  The call does
 * not allocate or synchronise and can be captured in a CUDA graph and replayed.
 * world <= 8.  Meant for messages up to about 1 MB; larger ones belong to the library
 * collectives (every rank sends its whole partial to every peer).
 */
size_t dxb_peer_allreduce_bytes(int world, int64_t capacity_elems);
int dxb_peer_allreduce(const void* partial, void* out, int64_t elems, void* const* peer_regions,
                       int64_t capacity_elems, int rank, int world, void* status,
                       void* cuda_stream);

/* Bytes of workspace dxb_wq_gemm needs for this problem on the current device.  For more
 * than 128 tokens this is what the one-launch plan over all token blocks needs; dxb_wq_gemm
 * also accepts the smaller amount a 128-token (and 96-token) problem asks for and then
 * launches block by block. */
size_t dxb_workspace_bytes(int M, int N, int K, int bits);

/*
 * Dense [K, N] bf16 weight, computed with the same bit-pattern arithmetic as the
 * GEMM kernel.  Replaces the reference's dequantize()
 * (python/dexter/ops/reference/gemm.py:51-73); used to check dequantisation
 * bit for bit.
 */
int dxb_dequantize(const void* qweight, const void* scales, const void* zeros, void* w_out, int N,
                   int K, int group_size, int bits, void* cuda_stream);

/* 1 when dxb_wq_gemm runs this shape on the tcgen05 kernel, 0 when it takes the
 * plain CUDA-core kernel (the counterpart of the reference's `accepts` shape
 * predicate, python/dexter/registry.py:58-60). */
int dxb_uses_tensor_cores(int M, int N, int K, int group_size, int bits);

/* Synchronises `cuda_stream` and returns the status word of `workspace`:
 * DXB_OK, or DXB_ERR_KERNEL_TIMEOUT if a kernel gave up on a wait. */
int dxb_read_status(void* workspace, void* cuda_stream);

/* Static, NUL-terminated description of a DXB_* code. */
const char* dxb_strerror(int code);

#ifdef __cplusplus
}
#endif

#endif /* DEXTER_B200_H_ */
