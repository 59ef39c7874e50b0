/* C ABI of the B200 (sm_100a) NVFP4 routed-expert path.
 *
 * Every entry point takes raw device pointers, plain integers and the CUDA stream to
 * launch on, allocates nothing, never synchronises, and returns 0 on success or a
 * negative code (ink_last_error() gives the message of the calling thread's last
 * failure). All are safe to call during CUDA-graph stream capture. "Reference" below
 * is Sourish07/Inkling-vs-Quad-RTX-3090s; each declaration names the interface it
 * stands in for.
 *
 * Conventions: activations and router weights are BF16 (passed as void*), expert
 * indices int64, pointer tables int64 device addresses laid out [expert][bank] with
 * the bank order of kernels/grouped_experts.py:9-22
 *   NVFP4: gate_up_proj, gate_up_proj_scale, gate_up_proj_scale2,
 *          down_proj,    down_proj_scale,    down_proj_scale2        (stride 6)
 * A zero first entry means "expert not on this rank / inactive": its routes are
 * skipped. NVFP4 banks: codes uint8 [rows, K/2] (two E2M1 codes per byte, low nibble
 * = even column), scales E4M3 bytes [rows, K/16], scale2 one FP32 read through its
 * pointer. gate_up rows interleave gate (even) and up (odd).
 */
#ifndef INKLING_B200_H_
#define INKLING_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct CUstream_st* ink_stream_t; /* == cudaStream_t */

/* Message of this thread's most recent failing call ("" if none). */
const char* ink_last_error(void);

/* Library/ABI version, bumped when a signature changes. */
int ink_abi_version(void);

/* ---------------------------------------------------------------- router ------
 * Replaces MyInklingTopkRouter.forward (my_inkling/model.py:311-350): BF16 logits =
 * x . W^T, score = bf16(sigmoid(logit)) + bias (FP32), top_k largest scores (ties:
 * lower expert id wins; emitted in descending score order), weights =
 * softmax(logsigmoid(selected + shared logits)) * route_scale * global_scale with the
 * BF16 rounding after every step that the reference's BF16 tensors impose.
 *
 *  x             BF16 [tokens, hidden]
 *  weight        BF16 [n_routed + n_shared, hidden]
 *  bias          FP32 [n_routed]
 *  global_scale  BF16 [1]
 *  routed_logits BF16 [tokens, n_routed] or NULL
 *  topk_weights  BF16 [tokens, top_k]; topk_indices int64 [tokens, top_k]
 *  shared_gammas BF16 [tokens, n_shared]
 *  workspace     ink_router_workspace_bytes(tokens, n_routed + n_shared) bytes,
 *                zero-filled once before first use (the kernel leaves it reusable)
 * Constraints: hidden % 8 == 0, top_k <= n_routed <= 512, top_k + n_shared <= 32.
 */
size_t ink_router_workspace_bytes(int tokens, int n_experts_total);
int ink_router_forward(const void* x, const void* weight, const float* bias, const void* global_scale,
                       float route_scale, int tokens, int hidden, int n_routed, int n_shared, int top_k,
                       void* routed_logits, void* topk_weights, int64_t* topk_indices,
                       void* shared_gammas, void* workspace, size_t workspace_bytes,
                       ink_stream_t stream);

/* The router for callers that cannot allocate device memory -- code that runs inside an
 * allocator callback or under a framework's memory plan that was fixed at start-up, a
 * host thread that must not take the allocator's lock, a process whose memory budget is
 * frozen once the model is resident. It has no counterpart in the reference. Same
 * arithmetic and outputs as ink_router_forward, but the kernel's scratch (block counter,
 * logits, selection scores: 35 072 bytes) is an array inside the library image instead
 * of a caller buffer, so every GPU the process uses holds those bytes until exit.
 * Limits: tokens <= 8 and n_routed + n_shared <= 544; anything larger is refused with an
 * error. It calls no cudaMalloc/cudaFree and no allocating library routine. The first call
 * on each device looks the array's device address up (cudaGetSymbolAddress); make that
 * first call outside stream capture. All calls share the one array and the kernel reads
 * what the previous call left there only after re-zeroing the counter, so calls must not
 * overlap on the GPU (issue them on one stream, or order them yourself): two calls in
 * flight at once race on the scratch. The address is looked up for the device that is
 * current at the call, so `stream` must belong to that device; and it is kept for the life
 * of the process, so the process must not reset the device (cudaDeviceReset) in between. */
int ink_router_forward_static(const void* x, const void* weight, const float* bias, const void* global_scale,
                              float route_scale, int tokens, int hidden, int n_routed, int n_shared, int top_k,
                              void* routed_logits, void* topk_weights, int64_t* topk_indices,
                              void* shared_gammas, ink_stream_t stream);

/* Router and expert plan in ONE launch (decode: tokens * top_k <= 512 routes); the
 * plan arguments are those of ink_expert_plan below. */
int ink_router_plan_forward(const void* x, const void* weight, const float* bias, const void* global_scale,
                            float route_scale, int tokens, int hidden, int n_routed, int n_shared, int top_k,
                            void* routed_logits, void* topk_weights, int64_t* topk_indices,
                            void* shared_gammas, void* workspace, size_t workspace_bytes,
                            const int64_t* sources, int64_t* pointers, int32_t* experts, int32_t* counts,
                            int32_t* rows, int start, int local, int stride, int capacity,
                            ink_stream_t stream);

/* ------------------------------------------------------------------ plan ------
 * Replaces the Triton kernel expert_plan (kernels/expert_planner.py:11-113) for a
 * placement in which every expert is resident (its LRU/slot outputs do not exist):
 *  counts per expert START+e, active experts compacted in ascending id into
 *  experts[] (-1 after) / counts[] (0 after), rows[g, :counts[g]] = ascending route
 *  numbers (route = token * top_k + choice), pointers[(start+e)*stride + b] =
 *  sources[e*stride + b] if the expert has routes else 0.
 * rows beyond counts[g] are left untouched, as in the reference.
 */
int ink_expert_plan(const int64_t* indices, const int64_t* sources, int64_t* pointers, int32_t* experts,
                    int32_t* counts, int32_t* rows, int start, int local, int stride, int routes,
                    int capacity, ink_stream_t stream);

/* ---------------------------------------------------------- decode GEMV ------
 * Replaces routed_decode (kernels/routed_decode.py:25-80) and its two CUDA kernels
 * gate_up / down_reduce (kernels/routed_decode.cu:137-173, :178-219):
 *   activated[route] = bf16(silu(gate) * up)        gate/up = scale2 * (W_gate_up . x)
 *   output[token]    = sum over choices of fp32(bf16(bf16(scale2 * (W_down . activated[route])) * w))
 * quantized = 1: NVFP4 banks as above. quantized = 0: the unquantised expert layer (the
 * reference's QUANT=0 build, kernels/routed_decode.cu:85-101): pointer table [expert][2] =
 * (gate_up_proj BF16 [2f, hidden], down_proj BF16 [hidden, f]), bank order of
 * expert_bank_names(False) (kernels/grouped_experts.py:9-22), same roundings with scale2 = 1.
 * output is fully overwritten; activated is scratch [tokens*top_k, intermediate].
 *  status: optional int32 device word; bit 0 is set when a route names an expert
 *          outside [0, max_expert] (the reference skips such routes silently).
 * Constraints: hidden and intermediate powers of two between 64 and 4096; top_k <= 30;
 * all buffers 16-byte aligned. An E4M3 scale byte 0x7F/0xFF decodes to NaN here (the
 * reference's table gives +-480); valid NVFP4 scales never use those codes.
 */
int ink_routed_decode(const void* x, const int64_t* indices, const void* weights, const int64_t* pointers,
                      void* activated, float* output, int tokens, int top_k, int hidden, int intermediate,
                      int max_expert, int quantized, int32_t* status, ink_stream_t stream);

/* Whole MoE layer at decode in two launches: the routed NVFP4 experts (as above) PLUS
 * the shared BF16 experts of MyInklingSharedExperts.forward (my_inkling/model.py:
 * 192-226; TP shard of my_inkling/tp_plan.py:128-146): per shared expert e
 *   act_e = bf16(bf16(bf16(silu(bf16 gate)) * bf16 up) * gamma_e),  down_e = bf16(W_down_e . act_e)
 * and output[token] = routed sum + sum_e fp32(down_e), FP32, fully overwritten: the
 * per-rank partial that one all-reduce then sums.
 *  shared_gate/up BF16 [n_shared, intermediate, hidden]; shared_down BF16 [n_shared, hidden, intermediate]
 *  gammas BF16 [tokens, n_shared]; shared_activated scratch BF16 [tokens*n_shared, intermediate]
 */
int ink_moe_decode(const void* x, const int64_t* indices, const void* weights, const int64_t* pointers,
                   void* activated, const void* shared_gate, const void* shared_up, const void* shared_down,
                   const void* gammas, void* shared_activated, float* output, int tokens, int top_k,
                   int n_shared, int hidden, int intermediate, int max_expert, int32_t* status,
                   ink_stream_t stream);

/* The two launches of ink_moe_decode on their own (same arguments): the gate/up half
 * writes activated / shared_activated, the down half reads them and writes output.
 * Lets a caller place other work between the halves, or time them apart. */
int ink_moe_gate_up(const void* x, const int64_t* indices, const void* weights, const int64_t* pointers,
                    void* activated, const void* shared_gate, const void* shared_up, const void* shared_down,
                    const void* gammas, void* shared_activated, float* output, int tokens, int top_k,
                    int n_shared, int hidden, int intermediate, int max_expert, int32_t* status,
                    ink_stream_t stream);
int ink_moe_down(const void* x, const int64_t* indices, const void* weights, const int64_t* pointers,
                 void* activated, const void* shared_gate, const void* shared_up, const void* shared_down,
                 const void* gammas, void* shared_activated, float* output, int tokens, int top_k,
                 int n_shared, int hidden, int intermediate, int max_expert, int32_t* status,
                 ink_stream_t stream);

/* ------------------------------------------------------------ layer glue ------
 * What sits either side of the MoE block in MyInklingDecoderLayer.forward
 * (my_inkling/model.py:672-675), reduced to its arithmetic skeleton for a stack of MoE
 * layers: the block's FP32 output is cast to BF16 and added to the residual stream
 * (BF16 add), and the sum is RMS-normalised for the next block exactly as the
 * reference's _rms_norm does (kernels/decode.py:36-43: FP32 reduction, the normalised
 * value rounded to BF16 BEFORE it is multiplied by the weight).
 *  partial   FP32 [tokens, hidden] (the all-reduced MoE output)
 *  residual  BF16 [tokens, hidden], updated in place to residual + bf16(partial)
 *  weight    BF16 [hidden]
 *  normed    BF16 [tokens, hidden]
 * Constraint: hidden % 8 == 0, hidden <= 16384.
 */
int ink_add_rmsnorm(const float* partial, void* residual, const void* weight, float eps, void* normed,
                    int tokens, int hidden, ink_stream_t stream);

/* The decode step of MyInklingShortConv (my_inkling/model.py:400-409), i.e. the Triton kernel
 * _short_conv (kernels/decode.py:65-146), which follows the MoE block as mlp_sconv with the
 * decoder residual (my_inkling/model.py:674-675): per channel c
 *   total = sum_{j < K-1} history[c][j+1] * taps[c][j] + x[c] * taps[c][K-1]      (FP32, tap order)
 *   history[c] <- (history[c][1..K-1], x[c])                                       (shifted in place)
 *   y[c] = bf16(total + x[c]);  with a residual: y[c] = bf16(fp32(y[c]) + residual[c])
 *  x         BF16 [batch, hidden], or with x_is_fp32 = 1 the block's all-reduced FP32 output
 *            [batch, hidden], which is rounded to BF16 first (my_inkling/offloaded_experts.py:314)
 *  taps      FP32 [hidden, kernel_size] (conv1d.weight [hidden, 1, K]; the checkpoint keeps it FP32)
 *  history   FP32 [batch, hidden, kernel_size], updated in place
 *  residual  BF16 [batch, hidden] or NULL;  y BF16 [batch, hidden]
 * kernel_size 2..4 (the model uses 4). */
int ink_short_conv(const void* x, int x_is_fp32, const float* taps, float* history, const void* residual,
                   void* y, int batch, int hidden, int kernel_size, ink_stream_t stream);

/* Decode attention with the learned relative-position bias, one query token per sequence: the static_decode
 * branch of MyInklingAttention.forward (my_inkling/model.py:533-612) from the normed query to the output of
 * scaled_dot_product_attention, with MyInklingRelativeLogits (my_inkling/model.py:112-133) and
 * MyInklingCache.decode_distance (my_inkling/cache.py:213-228) inside:
 *   distance[s] = position - s, in a sliding layer (window > 0) modulo the window (the cache is a ring)
 *   bias[s]     = bf16(r . proj[:, distance]) for 0 <= distance < rel_extent, else 0
 *   allowed[s]  = 0 <= distance <= position - pad_counts[b]
 *   full layers with n_floor > 0: tau = 1 + alpha * log(max((position + 1) / n_floor, 1)); q and bias times tau
 *   out = softmax(scale * q . K^T + bias, over the allowed slots) . V            (FP32 inside, BF16 out)
 *  q BF16 [batch, heads, head_dim] (after q_norm), r BF16 [batch, heads, d_rel], proj BF16 [d_rel, rel_extent],
 *  k_cache / v_cache BF16 [batch, kv_heads, slots, head_dim]: either the current token is already stored
 *  (ink_update_kv; new_k = new_v = NULL), or its key and value are given as new_k / new_v BF16 [batch, kv_heads,
 *  head_dim] and this call stores them at slot `position` (modulo the window) as well, saving the launch, position: device int64 scalar = tokens stored before this one (a CUDA graph advances it),
 *  pad_counts int64 [batch] or NULL, out BF16 [batch, heads, head_dim]. head_dim 64, 128 or 256.
 *  The cache is cut into groups of 64 slots, one block per (head, sequence, group); with more than
 *  one group the partial results pass through `workspace` (ink_decode_attention_workspace_bytes, 16-byte aligned) and
 *  the block that stores the last partial of a (sequence, head) joins them. The workspace must be ZERO before its first
 *  use (it starts with one arrival counter per (sequence, head)); every launch leaves the counters zero again, so the
 *  same workspace serves call after call on one stream. */
size_t ink_decode_attention_workspace_bytes(int batch, int heads, int head_dim, int slots);
int ink_decode_attention(const void* q, const void* r, const void* proj, void* k_cache, void* v_cache,
                         const int64_t* position, const int64_t* pad_counts, void* out, int batch, int heads,
                         int kv_heads, int head_dim, int d_rel, int rel_extent, int slots, int window, int n_floor,
                         float alpha, float scale, const void* new_k, const void* new_v, void* workspace,
                         size_t workspace_bytes, ink_stream_t stream);
/* The decode step of update_kv (kernels/decode.py:149-230): the new token's key and value, BF16
 * [batch, kv_heads, head_dim], into slot `position` (modulo the window in a sliding layer) of both caches. */
int ink_update_kv(const void* new_k, const void* new_v, void* k_cache, void* v_cache, const int64_t* position,
                  int batch, int kv_heads, int head_dim, int slots, int window, ink_stream_t stream);

/* ------------------------------------------------------ grouped projections ------
 * Replace the Triton kernels expert_gemm (kernels/grouped_experts.py:26-148) and
 * expert_reduce (:152-186) for more than a handful of tokens, on the tcgen05 tensor cores.
 * ink_expert_gemm: for every active group g (expert experts[g], routes rows[g, :counts[g]])
 *   projection 0: y[route, j] = bf16(silu(gate) * up), gate/up = even/odd rows of
 *                 W_gate_up[expert] . x[route / top_k]       (x BF16 [tokens, k], n = 2f rows)
 *   projection 1: y[route, :] = bf16(W_down[expert] . x[route])   (x BF16 [capacity, k], n = d rows)
 * FP32 accumulation in tensor memory. Weights enter the MMA as value * block scale in
 * FP16, which is exact, and the per-bank FP32 scale multiplies the accumulator; the
 * reference rounds value * (block scale * scale2) to BF16 first, so results agree to BF16
 * rounding of the weights, not bit for bit.
 *  input_rows  rows of x (tokens for projection 0, capacity for projection 1)
 *  groups      number of entries of experts/counts to visit (inactive ones cost nothing)
 *  scratch     ink_expert_gemm_scratch_bytes(input_rows) bytes
 * Constraints: NVFP4 banks; k a multiple of 128, at most 8192; n even.
 * ink_expert_reduce: output[token] += sum over choices of fp32(bf16(down[route] * w)),
 * skipping routes whose pointer row is zero; output FP32 [tokens, width], pre-zeroed by
 * the caller as in the reference (my_inkling/offloaded_experts.py:304).
 */
size_t ink_expert_gemm_scratch_bytes(int input_rows);
int ink_expert_gemm(const void* x, int input_rows, const int64_t* pointers, const int32_t* experts,
                    const int32_t* rows, const int32_t* counts, void* y, int capacity, int n, int k, int top_k,
                    int projection, int quantized, int groups, void* scratch, size_t scratch_bytes,
                    int32_t* status, ink_stream_t stream);
int ink_expert_reduce(const void* down, const int64_t* indices, const void* weights, const int64_t* pointers,
                      float* output, int tokens, int width, int top_k, int pointer_stride, int max_expert,
                      ink_stream_t stream);

/* The grouped projection on the BLOCK-SCALED tensor-core path (same reference kernel, same outputs as
 * ink_expert_gemm): the packed E2M1 codes of an expert's 128-row tile and their E4M3 block scales are the
 * M operand of tcgen05.mma.kind::mxf4nvf4.block_scale.block16 straight from the checkpoint layout -- no
 * conversion on the CUDA cores -- and the tokens routed to the expert are the N operand as four E2M1 digit
 * rows each (power-of-two block scales; exact to 2^-9 of the block's largest magnitude), eight tokens per
 * pass. Each active expert's bytes cross HBM once per eight of its tokens.
 *  bank_maps  device copy (128-byte aligned) of the 512 bytes ink_moe_stack_encode_banks wrote for this
 *             layer's banks, which must therefore be evenly spaced in memory; `start` is the expert id of
 *             the first bank the descriptors cover (experts[g] - start indexes them)
 *  pointers   as for ink_expert_gemm: the FP32 scale2 is read through it, a zero row skips the expert
 *  scratch    ink_expert_gemm_tc_scratch_bytes(input_rows, k) bytes: a kernel in front writes every input row's
 *             normaliser, digit rows and block scales there once; the main kernel reads them per expert tile
 * Constraints: n a multiple of 128, k a multiple of 256 up to 4096, groups <= 1024. */
size_t ink_expert_gemm_tc_scratch_bytes(int input_rows, int k);
int ink_expert_gemm_tc(const void* x, int input_rows, const void* bank_maps, const int64_t* pointers,
                       const int32_t* experts, const int32_t* rows, const int32_t* counts, void* y, int capacity,
                       int n, int k, int top_k, int projection, int groups, int start, void* scratch,
                       size_t scratch_bytes, int32_t* status, ink_stream_t stream);

/* ------------------------------------------------- whole stack, one launch ------
 * One decode token through n_layers MoE blocks in ONE persistent cooperative kernel:
 * per block the router (as ink_router_forward), the expert plan (resolved to bank
 * addresses on the device), the routed and shared experts (as ink_moe_decode), and --
 * with glue = 1 -- the residual add and RMS norm that ink_add_rmsnorm performs between
 * blocks. It replaces, for one token, the launches MyInklingMoE.forward issues per block
 * (my_inkling/model.py:361-374 through my_inkling/offloaded_experts.py:298-314).
 *
 *  layers       device array of n_layers descriptors, ink_moe_stack_layer_bytes() each:
 *               struct { const void *router_weight; const float *router_bias;
 *                        const void *global_scale; const int64_t *sources;    (sources: [experts][6])
 *                        const void *shared_gate, *shared_up, *shared_down; const void *norm_weight;
 *                        int64_t *topk_indices; void *topk_weights; void *gammas;    (optional outputs, may be null)
 *                        const void *bank_maps;   (device copy of ink_moe_stack_encode_banks' 512 bytes, or null)
 *                        float route_scale; int pad; }
 *               With bank_maps set in every layer the routed experts run on the tensor cores
 *               (tcgen05.mma kind::mxf4nvf4 on the packed codes and their block scales, no
 *               conversion); with null in every layer they run on the CUDA cores.
 *  x            BF16 [hidden]: input of the first block (x, residual_io, normed_out, partial_out and every
 *               layer's norm_weight are read and written 16 bytes at a time: 16-byte aligned)
 *  flags        bit 0 = glue, bit 1 = every layer carries bank_maps (run the routed experts on the tensor cores)
 *  glue = 0     n_layers must be 1; partial_out FP32 [hidden] receives the block's output
 *  glue = 1     residual_io BF16 [hidden] is the residual stream (updated in place),
 *               normed_out BF16 [hidden] the normalised output after the last block,
 *               partial_out the last block's FP32 output
 *  scratch      ink_moe_stack_scratch_bytes(...) bytes, ZERO-FILLED once before the first call and then
 *               left alone: its counters only grow (each launch reads how many launches came before;
 *               comparisons are modulo 2^32, so the count may wrap) and its hand-over words carry the
 *               tag of the launch and layer that wrote them. After a launch that reported a timed-out
 *               wait, zero it again before reuse.
 *  status       optional int32 word: bit 1 is set if a bounded wait inside the kernel gave up (the
 *               output of that launch is invalid; later launches on the same scratch give up too until
 *               it is zeroed again)
 * Built shapes (hidden, intermediate): (4096, 2048|1024|512|256), (2048, 256), (1024, 512);
 * experts <= 512, top_k <= 8, n_shared <= 2. The device must support cooperative launches.
 */
size_t ink_moe_stack_layer_bytes(void);
/* Encodes, on the host, the four TMA descriptors (4 x 128 bytes) through which the one-launch
 * kernel streams a layer's NVFP4 banks: gate/up codes [experts][2f][hidden/2], gate/up scales
 * [experts][2f][hidden/16], down codes [experts][hidden][f/2], down scales [experts][hidden][f/16],
 * each given by the device address of expert 0 and the byte distance between consecutive experts
 * (a multiple of 16; the banks of one kind must be evenly spaced, e.g. one allocation). Copy the
 * 512 bytes to 128-byte aligned device memory and point the layer's bank_maps at them. Has no
 * counterpart in the reference, which passes per-expert addresses (my_inkling/offloaded_experts.py:41-53). */
int ink_moe_stack_encode_banks(void* out_host_512, const void* gate_up_codes, uint64_t gate_up_codes_stride,
                               const void* gate_up_scales, uint64_t gate_up_scales_stride, const void* down_codes,
                               uint64_t down_codes_stride, const void* down_scales, uint64_t down_scales_stride,
                               int experts, int hidden, int intermediate);
/* Tracing (the reference's counterpart is utils/profiling.py:36-78): with the environment
 * variable INKLING_STACK_TRACE=1 every block stamps its phase boundaries with the global
 * nanosecond timer into the scratch at this byte offset, laid out
 * [n_layers][256 blocks][32 slots] of uint64 (slot meanings: enum TraceSlot in moe_stack.cu;
 * slots 0..23 are stamps, slots 24..31 SM clock cycles that consumer warp 0 waited for tiles or held
 * them in each section of the layer, and that producer lane 0 waited for its ring slot). */
size_t ink_moe_stack_trace_offset(int n_layers, int hidden, int intermediate, int experts, int n_shared,
                                  int top_k);
size_t ink_moe_stack_scratch_bytes(int n_layers, int hidden, int intermediate, int experts, int n_shared,
                                   int top_k);
int ink_moe_stack_decode(const void* layers, int n_layers, const void* x, void* residual_io, void* normed_out,
                         float* partial_out, int flags, float eps, int hidden, int intermediate, int experts,
                         int n_shared, int top_k, void* scratch, size_t scratch_bytes, int32_t* status,
                         ink_stream_t stream);

/* The same across `world` tensor-parallel ranks (one process per GPU, experts cut on the FFN
 * width, inputs and router replicated), with the all-reduce of every block done INSIDE the
 * kernel: it stands in for the per-block all-reduce of my_inkling/offloaded_experts.py:310 and
 * my_inkling/tp_plan.py:146 (kernels/paired_all_reduce.py:146-160). After the down projection
 * the block that owns a group of output rows stores its FP32 partial of them into slot `rank` of
 * every rank's region as 8-byte words {value, tag of this launch and layer} (plain stores over
 * NVLink into peer memory: no fence, no counter); the same block then polls its own region for
 * those rows from every rank, adds them in rank order -- so all ranks get the same bits -- and
 * publishes the sums to the blocks of its own GPU the same way. Every rank launches this with the
 * same arguments but its own layers/scratch and rank number.
 *  peer_regions  host array of `world` addresses: region r is rank r's buffer of
 *                ink_moe_stack_symmetric_bytes(n_layers, hidden, world) bytes as mapped into THIS
 *                process (peer access enabled; e.g. torch symmetric memory). Zero-filled once on
 *                every rank before any rank's first launch, then left alone like the scratch.
 * All ranks must issue the same sequence of launches (the tags are derived from the launch count),
 * and after a launch that timed out every rank zeroes scratch and region before any rank launches
 * again. Waits on other ranks are bounded like every other wait; no load with cluster scope
 * touches peer memory. */
size_t ink_moe_stack_symmetric_bytes(int n_layers, int hidden, int world);
int ink_moe_stack_decode_tp(const void* layers, int n_layers, const void* x, void* residual_io, void* normed_out,
                            float* partial_out, int flags, float eps, int hidden, int intermediate, int experts,
                            int n_shared, int top_k, void* scratch, size_t scratch_bytes, int rank, int world,
                            const uint64_t* peer_regions, int32_t* status, ink_stream_t stream);
/* How many SM clocks a wait inside the one-launch kernel may take before the launch gives up and
 * reports bit 1 of `status` (default 200 000 000, about a tenth of a second; at least 1000). Applies
 * to launches issued after the call, process-wide. Stands in for nothing in the reference, whose
 * kernels never wait on one another; it exists so that the give-up path can be exercised quickly. */
int ink_moe_stack_set_wait_limit(long long cycles);

#ifdef __cplusplus
}
#endif
#endif /* INKLING_B200_H_ */
