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
 * Launch order: the kernel is launched with programmatic stream serialisation, so it may
 * begin while the kernel before it on `cuda_stream` is still running.  It waits for that
 * kernel before it reads `x` or writes `out` / `workspace`, but it reads `qweight`, `scales`,
 * `zeros` and `bias` at once: these must be complete when the call is enqueued, i.e. they must
 * not be produced by the immediately preceding kernel of the same stream (weights are; a
 * caller that slices or copies weights per call must not).  DEXTER_B200_PDL=0 turns the
 * early start off.
 */
int dxb_wq_gemm(int bits, const void* x, int64_t ldx, const void* qweight, const void* scales,
                const void* zeros, const void* bias, void* out, int64_t ldo, int M, int N, int K,
                int group_size, void* workspace, size_t workspace_bytes, int max_ctas,
                void* cuda_stream);

/*
 * dxb_wq_gemm with options.  Replaces the same reference slot; each option stands for a
 * step the reference takes next to that slot:
 *   weight_layout  DXB_LAYOUT_DEXTER: `qweight` is the reference quantiser's tensor.
 *                  DXB_LAYOUT_B200 (int4 only): `qweight` is the output of dxb_relayout_w4,
 *                  the load-time repack the reference names as its own next step
 *                  ("pack into int32 words", README.md:147-150 of the reference).
 *   epilogue       DXB_EPILOGUE_GELU_TANH: tanh-GELU on the bf16 result (after the bias), what
 *                  the reference applies between the packed FFN linears
 *                  (python/dexter/models/dreamzero/model.py:279-285; oracle
 *                  python/dexter/ops/reference/gemm.py:92-100).
 *   max_ctas       as in dxb_wq_gemm.
 *   peer_*         peer_world > 1: this GEMM is one rank's K-shard of a row-parallel linear and
 *                  the sum over the ranks of one NVLink domain is part of the launch (the
 *                  reference has no tensor parallelism; this replaces a collective after the
 *                  call).  peer_regions[r] = rank r's region AS MAPPED IN THIS PROCESS (host array
 *                  of peer_world device pointers), each dxb_fused_reduce_bytes(world,
 *                  peer_capacity_elems) bytes of peer-mapped memory, zero-filled on every rank
 *                  before anyone's first call and used for nothing else.  Every rank must make
 *                  the same sequence of calls with the same M and N (K may differ), each on its
 *                  own GPU, one call in flight per region; M <= 128, M * N <= peer_capacity_elems,
 *                  a shape the tensor-core kernel takes (else DXB_ERR_UNSUPPORTED).  Every rank
 *                  passes the full `bias` (it is added after the sum) and receives the full
 *                  result in `out`: partial sums travel as bf16 and are added in fp32 in rank
 *                  order, so all ranks hold identical bits.  Waits for peers are bounded
 *                  (dxb_set_wait_limit_ms); on expiry DXB_ERR_KERNEL_TIMEOUT is left in the
 *                  workspace status word.  Plain peer stores and system-scope fences only.
 *   serialize      nonzero: plain stream order for this launch (no early start, see dxb_wq_gemm);
 *                  for a caller whose `qweight` / `scales` / `zeros` / `bias` were just written by
 *                  the preceding kernel of the stream.
 * `opts` may be NULL (all defaults).
 */
enum { DXB_LAYOUT_DEXTER = 0, DXB_LAYOUT_B200 = 1 };
enum { DXB_EPILOGUE_NONE = 0, DXB_EPILOGUE_GELU_TANH = 1 };
typedef struct dxb_gemm_opts {
  int weight_layout;
  int epilogue;
  int max_ctas;
  int peer_world;
  int peer_rank;
  void* const* peer_regions;
  int64_t peer_capacity_elems;
  int serialize;
} dxb_gemm_opts;

int dxb_wq_gemm_ex(int bits, const void* x, int64_t ldx, const void* qweight, const void* scales,
                   const void* zeros, const void* bias, void* out, int64_t ldo, int M, int N, int K,
                   int group_size, void* workspace, size_t workspace_bytes,
                   const dxb_gemm_opts* opts, void* cuda_stream);

/* Bytes of one rank's region for the fused sum over ranks (0 for an unsupported world size). */
size_t dxb_fused_reduce_bytes(int world, int64_t capacity_elems);

/*
 * Load-time repack of an int4 `qweight` [K/2, N] (python/dexter/quant.py:62-72 layout) into
 * the layout DXB_LAYOUT_B200 names, or back (`inverse` != 0).  Same shape and size; `out`
 * may equal `qweight`.  Inside every aligned block of 2 packed rows x 4 byte columns the 16
 * nibbles are regrouped so that one 32-bit word holds, for 4 columns, the two values of
 * consecutive k that the tensor-core operand pairs up; nothing moves between blocks, so
 * column slices (multiples of 4 columns) and row slices (multiples of 2 packed rows) of the
 * repacked tensor are the repacked slices.  K % 4 == 0 and N % 4 == 0 are required.
 */
int dxb_relayout_w4(const void* qweight, void* out, int K, int N, int inverse, void* cuda_stream);

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
 *   - all calls share the one array: the tile counters are cleared (cudaMemsetAsync on
 *     `cuda_stream`) at the start of every call, partial sums are overwritten before
 *     use; two calls that may run on the GPU at the same time (different streams, no
 *     ordering) race on it and must not be made;
 *   - a kernel that gave up on a bounded wait leaves DXB_ERR_KERNEL_TIMEOUT in the array's
 *     status word, which stays there until dxb_read_status(NULL, stream) has returned it.
 */
int dxb_wq_gemm_static(int bits, const void* x, int64_t ldx, const void* qweight,
                       const void* scales, const void* zeros, const void* bias, void* out,
                       int64_t ldo, int M, int N, int K, int group_size, void* cuda_stream);

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
/* The same for a call that caps the grid (`max_ctas` of dxb_wq_gemm); a cap can change how
 * tiles are split and with it the scratch needed.  dxb_wq_gemm also accepts the uncapped
 * amount: it then hands out whole tiles, which need no partial sums. */
size_t dxb_workspace_bytes_ex(int M, int N, int K, int bits, int max_ctas);

/*
 * Dense [K, N] bf16 weight, computed with the same bit-pattern arithmetic as the
 * GEMM kernel.  Replaces the reference's dequantize()
 * (python/dexter/ops/reference/gemm.py:51-73); used to check dequantisation
 * bit for bit.
 */
int dxb_dequantize(const void* qweight, const void* scales, const void* zeros, void* w_out, int N,
                   int K, int group_size, int bits, void* cuda_stream);
/* The same for a weight in `weight_layout` (DXB_LAYOUT_*). */
int dxb_dequantize_ex(const void* qweight, const void* scales, const void* zeros, void* w_out, int N,
                      int K, int group_size, int bits, int weight_layout, void* cuda_stream);

/* 1 when dxb_wq_gemm runs this shape on the tcgen05 kernel, 0 when it takes the
 * plain CUDA-core kernel (the counterpart of the reference's `accepts` shape
 * predicate, python/dexter/registry.py:58-60). */
int dxb_uses_tensor_cores(int M, int N, int K, int group_size, int bits);

/* Synchronises `cuda_stream` and returns the status word of `workspace`:
 * DXB_OK, or DXB_ERR_KERNEL_TIMEOUT if a kernel gave up on a wait.  `workspace` == NULL reads
 * the status word of the scratch built into the library (dxb_wq_gemm_static) and clears it. */
int dxb_read_status(void* workspace, void* cuda_stream);

/* Upper bound, in milliseconds, of a kernel's wait for another GPU (dxb_peer_allreduce and the
 * fused sum over ranks of dxb_wq_gemm_ex); process-wide, applies to later calls, about 1000 by
 * default.  No counterpart in the reference (which has no multi-GPU path). */
void dxb_set_wait_limit_ms(int ms);

/* Static, NUL-terminated description of a DXB_* code. */
const char* dxb_strerror(int code);

#ifdef __cplusplus
}
#endif

#endif /* DEXTER_B200_H_ */
