/* brokefish_b200 -- C ABI of the Blackwell (sm_100a) network evaluator.
 *
 * Drop-in boundary for the reference's evaluator extension: the pybind module
 * `brokefish_encoder` (csrc/encoder.cu:1905-1930) behind
 * `FusedEncoder.forward_full` (brokefish/nn/cuda_impl.py:487-504).  Plain pointers and
 * sizes only; no torch types.  Every function returns 0 on success or a negative
 * BF_E* code; `bf_last_error()` gives the text for the calling thread.
 *
 * Conventions
 *   - A handle belongs to one CUDA device.  Calls on one handle are not re-entrant.
 *   - `bf_forward*` take DEVICE pointers owned by the caller and enqueue one kernel on
 *     `stream` (a cudaStream_t passed as void*; NULL = the default stream).  They do
 *     not synchronise and allocate nothing.
 *   - `bf_forward_host` takes HOST pointers, copies in, runs, copies out and
 *     synchronises; it is the end-to-end call.
 *   - Every entry point that names a device (through a handle or a `device` argument) makes
 *     it current for the duration of the call and restores the caller's current device
 *     before it returns.
 *   - Every device-side wait in the kernel is bounded.  If one runs out, the kernel
 *     finishes with garbage outputs and a non-zero status word that `bf_status()`
 *     reads back after the caller's stream synchronisation.
 */
#ifndef BROKEFISH_B200_H
#define BROKEFISH_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define BF_OK 0
#define BF_EINVAL (-1)   /* bad argument, bad blob */
#define BF_ECUDA (-2)    /* a CUDA runtime call failed */
#define BF_ENOTSUP (-3)  /* network variant this build does not run */
#define BF_EDEVICE (-4)  /* a device-side bounded wait ran out */

#define BF_BLOB_MAGIC 0x38424642u /* "BFB8" */
#define BF_BLOB_VERSION 4u

/* GEMM selectors for bf_forward_capture. */
#define BF_OP_QKV 0 /* A: LN1 output s8 [rows,256]; acc [rows,768] in chunk order        */
#define BF_OP_OUT 1 /* A: attention output s8;       acc [rows,256]                       */
#define BF_OP_FF1 2 /* A: LN2 output s8;             acc [rows,1024]                      */
#define BF_OP_FF2 3 /* + hidden chunk c (3..6): A: hidden chunk u8 [rows,256]; acc [rows,256] */

typedef struct bf_handle bf_handle;

/* Library / build identification: "brokefish_b200 <version> sm_100a". */
const char* bf_version(void);

/* Text of the last error on the calling thread ("" if none). */
const char* bf_last_error(void);

/* Create an evaluator on CUDA device `device` from a packed weight blob (host or device
 * memory; layout in brokefish_b200/nn/pack.py; its header says which of the reference's kernel
 * modes it carries, in the reference's numbering (brokefish/nn/cuda_impl.py:95) — 3: int8 on all
 * four matmuls, 2: int8 FFN only, 4: int8 FFN and QKV, 1: e4m3 FFN with fp16 attention GEMMs,
 * 0: plain fp16 — and the matching kernel arm runs).  The blob is copied; the caller may free
 * it afterwards.  Replaces the weight slabs `FusedEncoder.__init__` uploads
 * (brokefish/nn/cuda_impl.py:228, 370-371, 382-406). */
int bf_create(const void* blob, size_t blob_bytes, int device, bf_handle** out);

/* Free a handle and everything it owns. */
int bf_destroy(bf_handle* h);

/* Number of layers / value rows / value mode recorded in the handle's blob. */
int bf_info(const bf_handle* h, int* n_layers, int* n_value, int* vmode);

/* Boards to logits, one launch.  Replaces `model_forward(..., debug_stage=0)`
 * (csrc/encoder.cu:1770-1876).
 *   boards  [n,32] u16 piece words      control [n] i16      rep [n] u8
 *   legal   [n,32] u64 or NULL: bit s of word p set <=> move p->s is legal; when given,
 *           illegal policy entries are written as fp16 -inf (0xFC00)
 *   policy  [n,32,64] fp16   promo [n,32,4] fp16   value [n] f32  (any may be NULL) */
int bf_forward(bf_handle* h, const uint16_t* boards, const int16_t* control,
               const uint8_t* rep, const uint64_t* legal, int n, void* policy, void* promo,
               float* value, void* stream);

/* Evaluate and expand in one launch: besides (optionally) the logits, write for every position
 * the edges of its search node and their priors, which the reference's search derives in a
 * kernel of its own from the logits (`Search._expand`, brokefish/search/torch_impl.py:962-1033;
 * `expand_node`, csrc/search.cuh:593-798).  `legal` [n,32]: bit s of word p says the piece in
 * slot p may move to square s.  Outputs, caller-owned device memory:
 *   prior  [n, e_cap] fp16   softmax over the node's candidates (policy logit, plus for a pawn
 *                            reaching its last rank log_softmax of its four promotion logits);
 *                            more than e_cap candidates: the e_cap largest stay (ties to the
 *                            earlier candidate) and are renormalised; zero beyond the edge count
 *   move   [n, e_cap] int16  slot * 64 + square | promotion type << 11, canonical order
 *   nedges [n] int32         edges written (0 for a position without a legal move)
 *   value  [n] fp32          as bf_forward; policy / promo may be NULL to skip the 4.3 KB per
 *                            position logit stream (when given, policy carries the legality AND)
 * e_cap is 1..255 (the reference's search uses 96).  `legal` may be NULL: the kernel then
 * generates the legal moves itself from the boards (bf_movegen's rules), policy must be NULL. */
int bf_forward_priors(bf_handle* h, const uint16_t* boards, const int16_t* control, const uint8_t* rep,
                      const uint64_t* legal, int n, int e_cap, void* prior, int16_t* move, int* nedges,
                      float* value, void* policy, void* promo, void* stream);

/* Evaluate a compacted leaf list: positions leaf_index[0 .. *leaf_count) of the staged arrays
 * (`boards`, `control`, `rep`, `legal` indexed by place), the count read ON THE DEVICE when the
 * kernel starts, so the caller needs no host synchronisation to know it.  `capacity` is the most
 * the list can hold (the grid is sized for it; a larger count is clamped, a negative one is 0);
 * CTAs beyond the count's tiles leave at once, so a short list runs short, and an int8 list of at
 * most one position per SM runs in the small-batch form (BF_OPT_ONE_BOARD).  Every output is
 * written at the position's own place in the staged arrays (policy [place,32,64], value [place],
 * prior [place,e_cap] ...); places not in the list are not touched.  Any of policy / promo /
 * value may be NULL; pass prior, move and nedges (all three, else all NULL) for the fused
 * expansion of bf_forward_priors.  Two list entries naming the same place race on its outputs
 * (same values).  No counterpart in the reference, whose search hands the evaluator all B staged
 * leaves whether active or not (brokefish/search/cuda_impl.py:304-320); this is the interface its
 * retrospective asks for (docs/journal/2026-08-09-kernel-design-retrospective.md, item 4). */
int bf_forward_leaves(bf_handle* h, const uint16_t* boards, const int16_t* control, const uint8_t* rep,
                      const uint64_t* legal, const int* leaf_index, const int* leaf_count, int capacity,
                      void* policy, void* promo, float* value, int e_cap, void* prior, int16_t* move,
                      int* nedges, void* stream);

/* Legal-move generation for `n` boards (device pointers): `mask` [n,32] 64-bit words, bit s of
 * word p set when the piece in slot p may legally move to square s (a promotion is one bit,
 * castling the king's two-square move, en passant a pawn's diagonal move to an empty square);
 * `in_check` [n] (may be NULL) for the side to move.  The engine contract of the reference's
 * `movegen` (brokefish/env/torch_impl.py:254-291; csrc/movegen.cuh): the input generator of the
 * evaluator's legality words and of the search's node masks.  One thread per board, one launch on
 * `stream`; needs no handle. */
int bf_movegen(int device, const uint16_t* boards, const int16_t* control, int n, uint64_t* mask,
               unsigned char* in_check, void* stream);

/* Play one move per board (device pointers): `move` [n] int32 = slot * 64 + target square, -1
 * leaves the board as it is; `promo` [n] int8 (may be NULL = queen) 0..3 = knight, bishop, rook,
 * queen.  Writes the new piece words (in place when boards_out == boards), the new control word
 * (side flipped; magnitude = the fifty-move counter, 1 after a capture or pawn move) and, when
 * non-NULL, `irreversible` [n] (capture, pawn move or a change of castling rights) -- the
 * reference's `step` (brokefish/env/torch_impl.py:412-548; `hash` non-NULL: the new position's key too;
 * csrc/movegen.cuh).  When `mask` is non-NULL the legal moves of the NEW position follow in the
 * same launch (bf_movegen's outputs), which is one ply of a self-play loop.  Moves are not
 * checked for legality.  One thread per board; needs no handle. */
int bf_step(int device, const uint16_t* boards, const int16_t* control, const int* move,
            const signed char* promo, int n, uint16_t* boards_out, int16_t* control_out,
            unsigned char* irreversible, uint64_t* mask, unsigned char* in_check, uint64_t* hash, void* stream);

/* Position keys for repetition detection: `hash` [n] of the given boards (bf_hash), or of the
 * boards after the move (the `hash` output of bf_step, may be NULL).  A key combines piece
 * (colour, type, square), side to move, castling rights and the file of an en passant capture
 * that is really available (a capturer stands beside the pawn and the capture does not expose
 * its king) -- the definition of the reference's `hash_position` (brokefish/env/torch_impl.py:
 * 374-401, 321-371).  The key values are this library's own, not the reference's table: only
 * their equality is meaningful, which is all repetition needs. */
int bf_hash(int device, const uint16_t* boards, const int16_t* control, int n, uint64_t* hash, void* stream);

/* The per-game repetition ring of the reference (brokefish/env/torch_impl.py:571-602): `ring`
 * [n,100] keys since the last irreversible move and `length` [n] int64, both updated in place.
 * bf_history_push records the position being LEFT (`hash` = its key, `irreversible` = what
 * bf_step said about the move; an irreversible move empties the ring); bf_repetition_count
 * gives how many times the position `hash` has occurred, counting the present one. */
int bf_history_push(int device, uint64_t* ring, long long* length, const uint64_t* hash,
                    const unsigned char* irreversible, int n, void* stream);
int bf_repetition_count(int device, const uint64_t* hash, const uint64_t* ring, const long long* length, int n,
                        int* count, void* stream);

/* Why each of `n` games is over, from a position's legal words, check flag, control word and
 * board (device pointers): `code` [n] uint8 = 1 checkmate, 2 stalemate, 3 fifty-move rule
 * (control magnitude >= 101), 4 threefold repetition (`rep_count` [n] from bf_repetition_count;
 * NULL skips the test), 5 insufficient material, 0 not over -- the first that applies; `result`
 * [n] int8 (may be NULL) = -1 for checkmate, else 0, from the side to move's point of view.  The
 * reference's `terminal` (brokefish/env/torch_impl.py:632-676, 604-629). */
int bf_terminal(int device, const uint64_t* mask, const unsigned char* in_check, const int16_t* control,
                const uint16_t* boards, const int* rep_count, int n, unsigned char* code, signed char* result,
                void* stream);

/* One ply of a uniform-random playout, in place (device pointers): from `mask` (the legal moves
 * of `boards`, bf_movegen's output) the floor(r[i] * count)-th legal move in (slot, square) order
 * is played with promotion type `promo[i]` (may be NULL = queen), and `mask` becomes the legal
 * moves of the new position; a board without legal moves is left alone.  `move` [n] int32 (may
 * be NULL) receives the move played or -1.  No single counterpart: the body of the reference's
 * random-playout loops (tests and benchmarks drive `movegen` + `play`,
 * brokefish/env/torch_impl.py:254-291, 412-548), here the generator of benchmark positions. */
int bf_random_ply(int device, uint16_t* boards, int16_t* control, uint64_t* mask, const float* r,
                  const signed char* promo, int n, int* move, void* stream);

/* The kernel's own quantisation ranges, for a host-side packer to check its constants against:
 * signed and unsigned int8 (127, 255) and the e4m3 operand range (8).  Replace the extension's
 * `fp8_q_max()` and `int8_q_max()` (csrc/encoder.cu:1906, 1926-1929). */
void bf_int8_q_max(int* signed_max, int* unsigned_max);
double bf_fp8_q_max(void);

/* Backbone only: activations in, activations out.  `x` [n,32,256] fp16 goes through the encoder
 * layers (no embedding, no final norm, no heads) and the residual stream after the last layer is
 * written to `y` [n,32,256] fp16 (y == x is allowed: a board's rows are read before they are
 * written); `alive` [n,32] int8 (may be NULL = all alive) masks dead tokens as attention keys.
 * Replaces `encoder_forward(y, weights, alive, n_layers, eps, 0)` (csrc/encoder.cu:1752-1767),
 * which the reference keeps on its fp16 arithmetic only; so does this: a handle whose blob
 * carries another arithmetic is refused with BF_ENOTSUP. */
int bf_forward_backbone(bf_handle* h, const void* x, const int8_t* alive, int n, void* y, void* stream);

/* Activations at an intermediate stage as [n,32,256] fp16.  Replaces
 * `model_forward(..., debug_stage=stage)` (csrc/encoder.cu:1315-1427, 1575-1598):
 * 9 embedding; layer 0: 1 LN1 out, 5/6/7 Q/K/V after bias, 4 attention out,
 * 2 residual after attention, 3 LN2 out; 8 final norm out. */
int bf_forward_stage(bf_handle* h, const uint16_t* boards, const int16_t* control,
                     const uint8_t* rep, int n, int stage, void* y, void* stream);

/* The same for any layer: stages 1-7 as above for layer `layer`, plus 10 = the residual
 * stream at the end of that layer; 8 and 9 ignore `layer`.  No counterpart in the
 * reference (its stage dumps stop at layer 0); used to locate a divergence by layer. */
int bf_forward_stage_at(bf_handle* h, const uint16_t* boards, const int16_t* control,
                        const uint8_t* rep, int n, int layer, int stage, void* y, void* stream);

/* Run the network and copy out, for one GEMM of one layer, the quantised A operand
 * bytes and the raw s32 accumulators the tensor cores produced.  This is what lets a
 * test recompute the exact integer product on the host (the method of the reference's
 * csrc/tests/tint8.cu:268-337).  `a_bytes` [n*32, 256] u8, `acc` [n*32, N] s32 with N by
 * `op` as listed at BF_OP_*. */
int bf_forward_capture(bf_handle* h, const uint16_t* boards, const int16_t* control,
                       const uint8_t* rep, int n, int layer, int op, uint8_t* a_bytes,
                       int32_t* acc, void* stream);

/* End-to-end call with HOST buffers (pinned for best speed): copies the inputs to the
 * device, runs the evaluator as a few launches of shrinking size (the last one a single wave of
 * tiles), copies each launch's three outputs back on a second stream while the next launch
 * computes -- only the last wave's copy is exposed -- and synchronises.
 * Device staging buffers are owned by the handle and grow to the largest `n` seen. */
int bf_forward_host(bf_handle* h, const uint16_t* boards, const int16_t* control,
                    const uint8_t* rep, const uint64_t* legal, int n, void* policy,
                    void* promo, float* value);

/* bf_forward_priors with HOST buffers, end to end like bf_forward_host: inputs (the legality
 * words included) go to the device, the evaluator runs wave by wave, and each wave's edge
 * lists and values come back on a second stream while the next wave computes; about 11 times
 * fewer bytes return to the host than with the logits (392 B per position at e_cap 96).  When
 * the outputs are pinned, device-mapped host memory the kernel writes them there directly. */
int bf_forward_priors_host(bf_handle* h, const uint16_t* boards, const int16_t* control, const uint8_t* rep,
                           const uint64_t* legal, int n, int e_cap, void* prior, int16_t* move, int* nedges,
                           float* value);

/* Options of a handle; no counterpart in the reference.
 *   BF_OPT_RSQRT_RN  0 (default): the LayerNorms take 1/sqrt from the hardware approximation,
 *                    as the reference kernel's `rsqrtf` does (csrc/encoder.cu:597), so outputs
 *                    follow that kernel bit for bit through the encoder body;
 *                    1: correctly rounded 1/sqrt, the only form a CPU restatement can
 *                    reproduce bit for bit (the parity tests against the numpy oracle use it). */
#define BF_OPT_RSQRT_RN 1
/*   BF_OPT_HOST_PLAN 0 (default): `bf_forward_host` sizes its launches by the device-to-host
 *                    rate its previous call measured: each launch as many times the next one as
 *                    copying a position out is faster than evaluating it (at most six times, a
 *                    GPU alone on its link), the last one a single wave; when copying is less than
 *                    1.5 times faster, equal launches of about two waves with the last wave
 *                    written straight into the caller's buffers (if pinned and device-mapped).
 *                    1: always the fast-link sizes; 2: always the equal launches.  Same outputs. */
#define BF_OPT_HOST_PLAN 4
/*   BF_OPT_ONE_BOARD k (default 1): an int8 evaluation of at most k boards per SM runs in the
 *                    small-batch form of the kernel -- one board per tile, its rows replicated in
 *                    the four lane quadrants, sixteen row warps per board instead of four, about
 *                    half the latency of a tile; 0 switches the form off.  Same outputs. */
#define BF_OPT_ONE_BOARD 5
int bf_set_option(bf_handle* h, int option, int value);

/* GB/s the first device-to-host copy of the last `bf_forward_host` call reached (0 before the
 * first call): what the plan of the next call is chosen by.  No counterpart in the reference. */
double bf_host_link_gbps(const bf_handle* h);

/* The launch sizes `bf_forward_host` uses for `n` positions on a GPU with `sm_count` SMs under
 * BF_OPT_HOST_PLAN `plan` when the measured copy rate is `gbps` (0: not measured yet): writes up
 * to 16 sizes, in launch order, summing to n, and returns how many; no GPU is touched.  No
 * counterpart in the reference. */
int bf_host_plan(int n, int sm_count, int plan, double gbps, int* sizes);

/* Read (and clear) the device status word; 0 = every launch since the last call ran
 * clean.  Synchronises the device. */
int bf_status(bf_handle* h, int* status);

/* Number of kernel launches this handle has enqueued. */
long long bf_launch_count(const bf_handle* h);

/* In-kernel phase accounting, the counterpart of the reference's `set_profile /
 * reset_profile / read_profile / profile_phases` hooks (csrc/encoder.cu:1110-1177,
 * 1886-1916).  While enabled, one thread of every CTA charges its clock cycles to the phase
 * it is in; `bf_profile_read` synchronises, returns the cycle sums since the last read (up
 * to 16 values, in the order `bf_profile_phases()` names them, comma separated) and clears
 * them.  Enabling or disabling also clears. */
int bf_profile(bf_handle* h, int enable);
int bf_profile_read(bf_handle* h, long long* cycles, int n);
const char* bf_profile_phases(void);

/* Evaluate without allocating anything.  No counterpart in the reference, which allocates
 * its slabs with torch: this exists for callers that must not (or cannot) allocate device
 * memory -- a worker inside a process whose GPU memory was partitioned up front, a plugin
 * host that forbids allocation after start-up -- and therefore cannot hold a `bf_handle`.
 *
 * The caller owns everything it passes: `blob_dev` is the packed weight blob already in
 * DEVICE memory (256-byte aligned, `blob_bytes` long), the other arguments are `bf_forward`'s.
 * The kernel's only other memory, its status word, is a 256-byte `static __device__` array
 * inside the library: every GPU that loads the library holds those 256 bytes until the
 * process exits, and nothing is ever cudaMalloc'ed or freed here.
 *
 * What it runs: int8 "all" blobs (arithmetic 3) without re-injection, any of the three value
 * heads.  A blob with another arithmetic or with re-injection is refused with BF_ENOTSUP and a
 * text that says which; such networks need a handle.
 *
 * Limits and rules
 *   - `n` above BF_NOALLOC_MAX_POSITIONS is refused (BF_EINVAL, text says so): split it.
 *   - The first call on a device resolves the array's device address, sets the kernel's
 *     shared-memory attribute and zeroes the status word; a call with a blob (pointer, size)
 *     the device has not seen reads and checks its 256-byte header (a synchronous copy) and
 *     remembers it.  Make such a call before any stream capture.
 *   - The remembered header is keyed on the blob's ADDRESS and SIZE only.  After writing new
 *     weights into the same device buffer (the rebuild-after-every-update pattern) call
 *     `bf_noalloc_forget(device)` first: without it the next call runs the new weights with the
 *     old header's value head, class count and epsilon.
 *   - All calls on a device share the one status word and it keeps what the last failing
 *     launch wrote until `bf_noalloc_status` reads it (which clears it).  Two launches that
 *     overlap on the GPU race on it: a time-out is still reported, but not whose it was.
 *   - Host threads may call concurrently, with the same or different blobs: the per-device
 *     record is read and replaced under a lock and each call launches from its own copy of the
 *     header.  Threads that alternate between two blobs on one device re-read a header on
 *     every switch.
 *   - The caller's current device is restored before the call returns. */
#define BF_NOALLOC_MAX_POSITIONS 1048576
int bf_forward_noalloc(int device, const void* blob_dev, size_t blob_bytes, const uint16_t* boards,
                       const int16_t* control, const uint8_t* rep, const uint64_t* legal, int n,
                       void* policy, void* promo, float* value, void* stream);

/* Drop what `bf_forward_noalloc` remembers about the blob last used on `device`, so that the
 * next call reads the header again.  Mandatory after re-packing into the same device buffer.
 * No counterpart in the reference. */
int bf_noalloc_forget(int device);

/* Synchronise `device` and read (and clear) the status word `bf_forward_noalloc` launches
 * share; 0 = clean.  No counterpart in the reference. */
int bf_noalloc_status(int device, int* status);

/* Measure what the tensor pipe sustains on `tcgen05.mma kind::i8` alone: one CTA per SM issues
 * `iters` groups of four M=128, N=256, K=32 MMAs on operands resident in shared memory, timed
 * with CUDA events (best of three after a warm-up).  `*tops` = int8 TOP/s of the whole device,
 * `*ms` (may be NULL) the duration.  The method of the reference's peak probe
 * (csrc/fp8_loop.cu; docs/ledger/perf.md:616-647), for the roofline's denominator. */
int bf_measure_i8_peak(int device, int iters, double* tops, double* ms);

/* The CUDA-core counterpart of bf_measure_i8_peak: elements per second, summed over the SMs, that
 * the evaluator's own element-wise device functions sustain in isolation (operands in shared
 * memory, sixteen warps per SM as in the evaluator, no tensor-memory loads, exchanges or
 * barriers).  `block`: 0 ff1 epilogue (descale, bias + ReLU, row maximum, u8 quantise), 1 descale
 * + bias to fp16 (QKV / out-projection epilogue), 2 ff2 step (descale + fused add to the fp16
 * running total), 3 norm statistics, 4 normalise + s8 quantise, 5 fp16 -> int8 quantise alone;
 * 6 and 7: block 0 again with eight and with thirty-two warps per SM; 8, 9, 10, 11: blocks 0, 4, 1
 * and 2 in a cheaper arithmetic that no longer reproduces the reference's bits (one combined
 * scale instead of two multiplies, the u8 requantisation done in fp16, the s8 quantisation fused
 * into the normalise) -- what a tolerance arm could save, measured before building one.
 * With the element counts of one position these give the time the reference's element-wise
 * arithmetic needs on this GPU however it is scheduled -- the second roof of this kernel.  No
 * counterpart in the reference beyond its wish for a benchmark that reports achieved against
 * measured ceilings (docs/journal/2026-08-09-kernel-design-retrospective.md, item 6). */
int bf_measure_elementwise(int device, int block, int iters, double* elements_per_s, double* ms);

/* Time-out self test; no counterpart in the reference.  A small kernel waits, through the same
 * bounded wait the evaluator's roles use, on an mbarrier that nothing arrives on.  The wait runs
 * out after its cycle limit (about 0.2 s), the kernel returns normally and `*status` receives
 * `code` (1..99), which is how a lost arrival would surface from the evaluator through
 * bf_status().  `waited_cycles` (may be NULL): [0] cycles the first waiter spent, [1] cycles a
 * second waiter spent after the flag was set (it returns at once).  Nothing faults or hangs. */
int bf_selftest_timeout(int device, int code, int* status, long long* waited_cycles);

/* Tensor-core self test (no network): one 128-row tile times a packed weight tile.
 *   mode 0: s8 x s8, N=128, K=256     mode 1: u8 x s8, N=128, K=256
 *   mode 2: s8 x s8, N=192, K=256     mode 3: f16 x f16 -> f32, N=96, K=256
 *   mode 4: e4m3 x e4m3 -> f32, N=128, K=256
 *   a        device, [128, K] row-major (1 byte or 2 bytes per element)
 *   w_image  device, K/ (128 B) stage images of [N, 128 B] (pack.py: sw128_image)
 *   out      device, [128, N] s32 (modes 0-2) or f32 (modes 3, 4)
 * Follows the exact-integer method of the reference's csrc/tests/tint8.cu:268-337. */
int bf_selftest_umma(int device, int mode, const void* a, const void* w_image, void* out);

#ifdef __cplusplus
}
#endif
#endif /* BROKEFISH_B200_H */
