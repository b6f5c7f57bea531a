/*
 * crusader_b200 — training-step executor over the C ABI of crusader_b200.h.
 *
 * Replaces the inner loop of the reference's Sequential::train (seann/containers/Sequential.cu:43-104:
 * forward / backward / learn) for the ResNet family of the specification, keeping the reference's training
 * semantics: gradients summed over the batch, loss gradient softmax - onehot (seblas/operations/cuLoss.cu:231),
 * BatchNorm per (c,h,w) position (cuBatchNorm.cu:14-61), residual blocks as in archive/Resnet56:8-15, Momentum with
 * multiplicative weight decay (seann/optimizers/Optimizers.cu:17-22).
 *
 * Parameters, gradients and momentum are three flat caller-owned device buffers with one layout (cbt_param_entry),
 * so a data-parallel caller sum-allreduces the one gradient buffer between cbt_backward and cbt_update.
 */
#ifndef CRUSADER_B200_TRAIN_H
#define CRUSADER_B200_TRAIN_H

#include "crusader_b200.h"

#ifdef __cplusplus
extern "C" {
#endif

typedef struct cbt_model cbt_model;

/* ResNet with 6*blocks_per_stage + 2 layers (9 -> ResNet-56) on batch x 3 x image_hw x image_hw inputs. */
int cbt_resnet_create(cbt_model** out, cb_ctx* ctx, int batch, int blocks_per_stage, int image_hw, int classes);
/* DenseNet-BC with growth k and `layers` bottleneck layers per dense block (k = 12, layers = 16: DenseNet-BC-100),
 * compression 0.5, 2x2 average-pool transitions, on batch x 3 x image_hw x image_hw inputs. */
int cbt_densenet_create(cbt_model** out, cb_ctx* ctx, int batch, int growth, int layers, int image_hw, int classes);
int cbt_destroy(cbt_model* m);
const char* cbt_last_error(const cbt_model* m);

/* Flat parameter layout: total floats, number of tensors, and entry i = (offset, size, is_weight,
 * kind: 0 conv filter, 1 BN gamma, 2 BN beta, 3 FC weight, 4 FC bias, dims[4]). */
long long cbt_param_count(const cbt_model* m);
int cbt_param_entries(const cbt_model* m);
int cbt_param_entry(const cbt_model* m, int i, long long* offset, long long* size, int* is_weight, int* kind, int* dims);
int cbt_op_count(const cbt_model* m);

/* Binds the flat device buffers (cbt_param_count floats each, 16-byte aligned; gradients start at zero). */
int cbt_bind(cbt_model* m, float* params, float* grads, float* momentum);

/* Must be called after the caller wrote to the bound parameter buffer by any route other than cbt_update (initial
 * values, a checkpoint, a broadcast between replicas): the executor keeps packed copies of the convolution filters
 * from one update to the next (cb_conv_cache_filters) and re-makes them here. */
int cbt_params_changed(cbt_model* m);

/* One training step in three asynchronous parts on the context's stream. */
int cbt_forward(cbt_model* m, const float* images, const float* labels_onehot);
int cbt_backward(cbt_model* m);
int cbt_update(cbt_model* m, float lr, float beta, float l2);

/* The convolution weight gradients of cbt_backward run on `n` CUDA streams of the executor's own (0..4; 0: on the
 * context's stream). Only the update needs them, so they fill the SMs that the chain of data-gradient and BatchNorm
 * kernels leaves idle; each forks where its layer's output gradient is complete and joins before cbt_backward's work
 * ends, so callers see no difference in ordering. Default: environment variable CBT_WGRAD_STREAMS, else 2. Not while
 * the stream is being captured. cbt_side_launches counts the launches made there (cb_launch_count does not). */
int cbt_set_wgrad_streams(cbt_model* m, int n);
long long cbt_side_launches(const cbt_model* m);

/* BatchNorm statistics per group of batch / groups consecutive samples instead of over the whole batch (default 1).
 * On one GPU, G groups compute exactly what G data-parallel ranks compute on their shards of the same batch. */
int cbt_set_bn_groups(cbt_model* m, int groups);

/*
 * Data-parallel training, one process per GPU (the batch sharded by rank, weights replicated; the reference trains on
 * one GPU only, seann/containers/Sequential.cu:107-163). Rank 0 obtains a 128-byte rendezvous id with
 * cbt_dp_unique_id and hands it to the other ranks over any host channel; every rank then calls cbt_dp_init
 * (collective). From then on cbt_backward sum-allreduces the flat gradient buffer over the ranks with NCCL, in
 * `buckets` contiguous ranges (1..8; the range of the first layers, which is ready last, is the smallest and each
 * next one twice as large), each issued on a communication stream as soon as the backward pass has
 * produced its last gradient, so the exchange overlaps the rest of the backward pass; everything queued on the
 * context's stream after cbt_backward sees the summed gradients. Every rank then applies the same cbt_update, so the
 * replicas stay bit-identical without a broadcast. NCCL is loaded at run time (libnccl.so.2); CB_EUNSUPPORTED without it.
 * A CUDA graph that captured cbt_backward of a data-parallel model must be destroyed before cbt_destroy: NCCL keeps
 * a communicator alive, and ncclCommDestroy waiting, for as long as a graph holds one of its collectives.
 */
int cbt_dp_unique_id(char* id128);
int cbt_dp_init(cbt_model* m, const char* id128, int world, int rank, int buckets);
int cbt_dp_world(const cbt_model* m);

/* on = 1: store BatchNorm's two parameter gradients in each other's slot, which is what the reference's operand does
 * (seann/operands/seblas/BatchNorm.cu:24 passes beta's and gamma's gradient tensors to seblas::batchNormParamGrads in
 * swapped order); for step-by-step comparisons with the reference's own operand graph. Default 0: the right slots. */
int cbt_set_reference_bn_grad_order(cbt_model* m, int on);

/*
 * The reference's model files (.crseq; writer seio/modelcache/codec.cu:8-39 saveSequence, reader :41-97 loadSequence,
 * records seann/operands/<operand>::encodeInfo / encodeNetParams and seann/containers/NetParam.cuh:45-72), for ResNet
 * models, whose operand list is the reference's own (cuConv2D, BatchNorm, ReLU, ShortcutEndpoint pairs with the 1x1
 * projection as branch operand, GlobalAvgPool, Linear, Softmax). cbt_save_crseq writes the bound parameters in that
 * format (replacing the file; block uuids 1, 2, ...); cbt_load_crseq checks that the file describes this very network
 * and loads its parameters, returning the file's epoch id. Both wait for the context's stream. CB_EUNSUPPORTED for
 * other model families, CB_EINVAL with cbt_last_error naming the first difference for a file of another network.
 */
int cbt_save_crseq(cbt_model* m, const char* path, unsigned epoch);
int cbt_load_crseq(cbt_model* m, const char* path, unsigned* epoch);

/* Mean cross-entropy per sample of the last forward pass (synchronises the stream), as Sequential::train logs it. */
int cbt_loss(cbt_model* m, float* loss_mean);
/* Device pointers for tests: value (grad = 0) / gradient (grad = 1) of tensor id; -1 = logits, -2 = softmax. */
float* cbt_tensor_ptr(cbt_model* m, int id, int grad);
float* cbt_loss_ptr(cbt_model* m);
int cbt_copy_loss(cbt_model* m, float* dst);
int cbt_copy_tensor(cbt_model* m, int id, int grad, float* dst, long long n);

#ifdef __cplusplus
}
#endif
#endif /* CRUSADER_B200_TRAIN_H */
