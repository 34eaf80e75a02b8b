/*
 * mt_capi.h -- C driver entry points of libmicrotorch, the C++ host library that
 * holds the tape (microtorch::backward / checkpoint), the ops, the layers and the
 * model families. They let a host language without a C++ binding (the Python
 * benchmark and test drivers use ctypes) build a model, run the checkpointed
 * training step and read results back. Every call returns 0 on success; on failure
 * the message is available from mt_last_error(). Pointers ending in _h are host
 * pointers.
 *
 * The step these entries drive is the reference's own loop -- zero_grad, forward,
 * ops::cross_entropy, backward, clip, AdamW::step -- as written in its
 * tests/test_checkpointing.cpp:45-58 and tools/mtstudio.cpp:456-480.
 */
#ifndef MT_CAPI_H_
#define MT_CAPI_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

const char* mt_last_error(void);

/* Selects GPU `device`, sets the compute dtype (0 = fp32, 1 = bf16 activations and
 * GEMM operands with fp32 master weights, gradients of parameters and accumulation). */
int mt_init(int device, int dtype);
/* Run all work on this cudaStream_t (NULL: the library's own stream). */
int mt_set_stream(void* cuda_stream);
int mt_sync(void);

/* spec: "key=value;key=value;..." with keys
 *   family   llama | gpt2 | flex
 *   vocab d layers heads kv_heads dff nctx theta tie rope_all qlora rank alpha seed
 *   norm (layernorm|rmsnorm)  act (gelu|relu|swiglu)  pos (learned|sinusoidal)   [flex]
 *   ckpt (0|1: per-block activation checkpointing)
 *   pack (0|1, default 1: parameters, gradients and bf16 shadows in flat buffers)
 * Unknown keys are an error. */
int mt_model_create(const char* spec, void** model_h);
int mt_model_destroy(void* model);
int mt_model_set_checkpoint(void* model, int on);
/* rows > 0: the vocabulary projection and the cross entropy run fused over chunks of that many
 * rows, so the [tokens, vocab] logits never exist as a whole (default: about 2^29 logits per chunk,
 * i.e. 16384 rows for a 32000-word vocabulary, 3072 for 151936). rows = 0: the two
 * separate ops of the reference (src/llama.cpp:85-88 then src/ops.cpp:350-376). */
int mt_model_set_loss_chunk(void* model, int64_t rows);

int mt_model_num_params(void* model, int64_t* n_h);
int mt_model_param_info(void* model, int64_t index, char* name_h, size_t cap, int64_t* rows_h, int64_t* cols_h);
int mt_model_param_get(void* model, int64_t index, float* out_h);
int mt_model_param_set(void* model, int64_t index, const float* in_h);
/* *has_grad_h = 0 when the parameter never received a gradient (out_h untouched). */
int mt_model_grad_get(void* model, int64_t index, float* out_h, int* has_grad_h);

/* One pass: zero_grad, forward over `n` token ids (B sequences of seq_len stacked;
 * seq_len = 0 means one sequence), mean cross entropy against targets, scaled by
 * loss_scale, and -- when do_backward != 0 -- the reverse pass. *loss_h receives the
 * UNSCALED mean loss (read back after the backward was enqueued). */
int mt_model_step(void* model, const int32_t* ids_h, const int32_t* targets_h, int64_t n, int64_t seq_len,
                  float loss_scale, int do_backward, float* loss_h);
/* Variables alive between forward and backward of the last mt_model_step (the
 * reference's memory receipt for checkpointing, include/microtorch/autograd.hpp:61-64). */
/* ---- one Llama block on its own (spec family=block; keys d, heads, kv_heads, dff, theta,
 * rope_all, seed, ckpt, pack): the single-block microbenchmark configuration. The block is
 * include/microtorch/llama.hpp:14-33 / src/llama.cpp:9-60 of the reference; checkpointing is
 * checkpoint(fn, x) around its forward (src/autograd.cpp:68-102). Parameters are reached
 * through the mt_model_param_* / mt_model_grad_get calls above.
 * set_input uploads x [rows, d] and the upstream gradient dy [rows, d] (host fp32; rows =
 * sequences x seq_len); forward runs y = block(x), keeping only x when checkpointing is on;
 * backward seeds y with dy: recompute + backward when checkpointed. */
int mt_block_set_input(void* model, const float* x_h, const float* dy_h, int64_t rows, int64_t seq_len);
int mt_block_forward(void* model);
int mt_block_backward(void* model);
int mt_block_output(void* model, float* y_h);          /* between forward and backward */
int mt_block_input_grad(void* model, float* dx_h);     /* after backward */

int mt_model_live_after_forward(void* model, int64_t* n_h);

/* AdamW with the reference's defaults unless set (lr 1e-3, betas 0.9/0.999, eps 1e-8, wd 0.01). */
int mt_model_set_adamw(void* model, float lr, float beta1, float beta2, float eps, float weight_decay);
int mt_model_optimizer_step(void* model);

/* Checkpoint files in the safetensors layout of the reference (src/safetensors.cpp:12-94: 8-byte
 * little-endian header length, JSON header, raw fp32 tensors in sorted name order, header padded
 * to 8 bytes). mt_model_save writes every parameter under its mt_model_param_info name as F32
 * [rows, cols] -- a file the reference's load_safetensors reads -- and, when optimizer_path is not
 * null, a second file beside it with the AdamW state ("m.<name>", "v.<name>", and "t" = [low 24
 * bits, high bits] of the step count), which the reference does not save
 * (tools/mtstudio.cpp:437-441). mt_model_load is the inverse (either path may be null); it
 * also accepts BF16 tensors, checks every name and shape before changing anything, and a run
 * restored from both files continues bit-identically. mt_safetensors_copy loads a file and writes
 * it back (no GPU needed): the loader's rules -- rank > 2 skipped, "transformer." stripped,
 * "__metadata__" ignored, [n] -> [1, n] -- applied to any safetensors file. */
int mt_model_save(void* model, const char* weights_path, const char* optimizer_path);
int mt_model_load(void* model, const char* weights_path, const char* optimizer_path);
int mt_safetensors_copy(const char* in_path, const char* out_path, int64_t* n_loaded_h, int64_t* n_skipped_h);
/* QLoRA models (spec qlora=1): replaces the frozen base -- the seven projections of every block,
 * the embedding and the norm gains -- by the tensors of a dense model's weights file (F32 or
 * BF16 safetensors, that model's parameter names); the projections are quantised to Q8_0 on the
 * device, as the reference builds its QLoRA layers from fp32 weights (src/quant.cpp:102-110).
 * Names and shapes are all checked first. The LoRA matrices are left as they are. */
int mt_model_load_base(void* model, const char* weights_path);
/* The other direction: writes the weights file of the equivalent dense model, every projection
 * merged as deq(Wq) + (alpha / r) A B in fp32 on the device (the reference's merged_weight,
 * src/quant.cpp:82-89), under the dense model's names. */
int mt_model_save_merged(void* model, const char* weights_path);
/* GGUF (version 3) export with the byte layout of the reference's exporter
 * (include/microtorch/gguf.hpp:58-66, src/gguf.cpp:27-166): llama.* metadata, token_embd /
 * blk.N.* / output_norm (/ output) tensors as F32, data aligned to 32 bytes.
 * mt_model_export_gguf writes a llama-family model (a QLoRA model with its adapters merged).
 * mt_gguf_export_llama converts a safetensors file without a GPU: spec keys name, arch, ctx, d,
 * layers, dff, heads, kv_heads, vocab, eps, theta, in_out (1: projections stored [in, out] and
 * transposed on export; 0: stored [out, in] as in HF checkpoints); tokens_path (may be null)
 * names a text file with one token per line for the tokenizer block; *n_unmapped_h receives the
 * number of tensors of the file that have no place in the layout. */
int mt_model_export_gguf(void* model, const char* gguf_path, const char* name, int64_t context_length);
int mt_gguf_export_llama(const char* weights_path, const char* gguf_path, const char* spec, const char* tokens_path,
                         int64_t* n_unmapped_h);

/* Gradient accumulation over micro-batches (the reference's trainer loop,
 * tools/mtstudio.cpp:456-474: zero_grad once, `accum` backward passes pre-scaled by 1/accum,
 * one optimizer step). With accumulate on, mt_model_step no longer clears the gradients it
 * finds; the caller clears them with mt_model_zero_grad before the first micro-step and passes
 * loss_scale = 1/accum. A data-parallel launcher all-reduces on the last micro-step only. */
int mt_model_set_accumulate(void* model, int on);
int mt_model_zero_grad(void* model);

/* Optimizer state for checkpoint / resume. The reference saves weights only
 * (tools/mtstudio.cpp:437-441), so there a resumed run starts its moments from zero; with
 * these entries a run restored from (parameters, step count, both moments of every parameter)
 * continues bit-identically. `index` is the index of mt_model_param_info; m_h / v_h hold
 * rows*cols floats on the host. Moments read as zero before the first optimizer step. */
int mt_model_optimizer_steps_get(void* model, int64_t* t_h);
int mt_model_optimizer_steps_set(void* model, int64_t t);
int mt_model_optimizer_state_get(void* model, int64_t index, float* m_h, float* v_h);
int mt_model_optimizer_state_set(void* model, int64_t index, const float* m_h, const float* v_h);
/* ops::clip_grad_norm (src/ops.cpp:1046-1064): global L2 norm of all gradients, summed in
 * double on the device; when it exceeds max_norm every gradient is scaled by max_norm / norm.
 * *norm_h receives the norm before clipping. */
int mt_model_clip_grad_norm(void* model, float max_norm, float* norm_h);
/* The same op on n host arrays [rows_h[i], cols_h[i]] taken as the gradients of n variables:
 * uploaded, clipped on the device, written back in place. */
int mt_clip_grad_norm_arrays(int n, const int64_t* rows_h, const int64_t* cols_h, float* const* grads_h, float max_norm,
                             float* norm_h);

/* Gradient ranges for data parallelism: bucket i < n-1 is the contiguous fp32 gradient
 * range of transformer block i; the last bucket holds everything else (embeddings,
 * final norm, head). Needs pack=1. */
int mt_model_num_buckets(void* model, int64_t* n_h);
int mt_model_bucket(void* model, int64_t index, void** ptr_h, int64_t* count_h);
/* cb(k, user) runs on the calling thread right after the backward of the k-th
 * checkpointed segment finished being enqueued (k counts from 0 per step, in reverse
 * block order: k = 0 is the last block). NULL removes the hook. */
typedef void (*mt_segment_cb)(int, void*);
int mt_set_segment_hook(mt_segment_cb cb, void* user);

/* Data parallelism inside the library (no Python, no torch.distributed on the data path): the
 * gradient exchange of microtorch/dp.hpp over the collective group of libpk (NCCL). Rank 0 draws
 * the 128-byte id with mt_dp_unique_id and the launcher hands it to every rank; mt_dp_init builds
 * the communicator on the model's GPU (max_ctas > 0 caps NCCL's CTAs, 0 = its default) and
 * installs the exchange as the segment hook (it replaces a hook set with mt_set_segment_hook):
 * from then on every mt_model_step starts the all-reduce of a block's gradients as that block's
 * backward is enqueued. The caller scales the loss by 1 / world (loss_scale of mt_model_step),
 * calls mt_dp_finish after the (last) backward and before mt_model_optimizer_step -- it sends
 * the remaining ranges and orders the compute stream behind all transfers, without blocking
 * the host -- and, under gradient accumulation, mt_dp_enable(model, 0) for all but the last
 * micro-batch. A model with less than 32 MiB of gradients (LoRA adapters) is sent as one flat
 * buffer in one collective. mt_dp_wait_host blocks until the transfers are done and fails after
 * the time limit (mt_dp_set_timeout, default 30 s), aborting the communicator: a rank that
 * died is noticed there, not by hanging. Needs pack=1. */
int mt_dp_unique_id(void* id_h, size_t cap);
int mt_dp_init(void* model, const void* id_h, int rank, int world, int max_ctas);
int mt_dp_enable(void* model, int on);
int mt_dp_finish(void* model);
int mt_dp_wait_host(void* model);
int mt_dp_set_timeout(void* model, double seconds);
/* Gradient bytes up to which the whole buffer is sent as one collective (default 32 MiB; 0: always
 * one collective per block, started during the backward pass). */
int mt_dp_set_flat_threshold(void* model, int64_t bytes);
int mt_dp_stats(void* model, int64_t* launches_last_step_h, int* single_collective_h);
int mt_dp_destroy(void* model);

/* out_h[0..5] = activation bytes in use, activation peak, persistent in use, persistent
 * peak, bytes reserved from the driver, number of driver allocations. */
int mt_mem_stats(uint64_t* out_h);
/* What was live at the activation high-water mark (since mt_reset_peak): up to `cap` pairs
 * (block size in bytes, number of blocks) in ascending size order; *n_h = number of distinct
 * sizes. Sizes identify the tensors of a step ([tokens, d], [tokens, d_ff], ...). */
int mt_mem_peak_blocks(uint64_t* sizes_h, uint64_t* counts_h, int cap, int* n_h);
int mt_reset_peak(void);
int mt_empty_cache(void);
int mt_live_variables(int64_t* n_h);

#ifdef __cplusplus
}
#endif
#endif /* MT_CAPI_H_ */
