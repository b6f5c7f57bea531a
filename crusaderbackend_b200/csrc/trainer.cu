// A compact training-step executor for the models of the specification (ResNet-56 and its shallower
// siblings), written on top of the C ABI of this library. It replaces the inner loop of the reference's
// Sequential::train (seann/containers/Sequential.cu:43-104: forward, backward, learn) for these models, with the
// reference's training semantics:
//   * gradients are summed over the batch (no 1/N), the loss gradient is softmax - onehot
//     (seblas/operations/cuLoss.cu:231-234) and the reported loss is sum(-log(y + 1e-10) * label) / batch
//     (cuLoss.cu:220-229 with seann/containers/Sequential.cu:125-130);
//   * BatchNorm normalises every (c,h,w) position over the batch (seblas/operations/cuBatchNorm.cu:14-61);
//   * a residual block is  x -> conv-BN-ReLU-conv-BN -> (+ shortcut) -> ReLU, the shortcut being the identity or a
//     bare 1x1 stride-2 convolution (archive/Resnet56:8-15, :96);
//   * Momentum: w *= (1 - l2) on weights, m = beta m + (1 - beta) g, w -= lr m, g = 0
//     (seann/optimizers/Optimizers.cu:17-22, seblas/operations/cuOptim.cu:38-46).
// Parameters, gradients and momentum live in three flat caller-owned device buffers (same layout), so a
// data-parallel caller sum-allreduces ONE gradient buffer between cbt_backward and cbt_update.
#include <dlfcn.h>

#include <algorithm>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>

#include "cb_internal.h"

namespace {

enum OpKind { OP_CONV, OP_BN, OP_RELU, OP_ADD, OP_GAP, OP_LINEAR, OP_SOFTMAX_CE, OP_CONCAT, OP_AVGPOOL, OP_HEAD };

struct TensorBuf {
    int n = 0, c = 0, h = 0, w = 0;
    float* a = nullptr;   // value
    float* d = nullptr;   // gradient (allocated lazily for tensors that need one)
    // A view is a channel range [c_off, c_off + c) of a wider tensor `view_of` (a DenseNet block buffer): it shares that
    // tensor's memory, so its samples are the parent's sample size apart.
    int view_of = -1, c_off = 0;
    long long bstride = 0;  // floats between consecutive samples; 0 = dense (c * h * w)
    long long size() const { return (long long)n * c * h * w; }
    long long sample() const { return (long long)c * h * w; }
};

struct Op {
    OpKind kind;
    int in0 = -1, in1 = -1, out = -1;  // tensor ids
    // conv
    int oc = 0, f = 0, stride = 1, pad = 0;
    long long w_off = -1, b_off = -1;   // offsets into the flat parameter buffer (conv filter / BN gamma / FC weight; BN beta / FC bias)
    int xhat = -1;                      // BN: tensor id of x-hat
    bool in0_grad_accumulate = false;   // backward adds into in0's gradient instead of overwriting it
    bool in1_grad_accumulate = false;   // likewise for the second input (shortcut of a fused BatchNorm-add-ReLU)
    bool relu = false;                  // BN / ADD: a ReLU is folded into this op (out is the activated tensor)
    int pooled = -1, logits = -1, probs = -1;  // HEAD: tensors holding the pooled features, logits and softmax
};

// The few NCCL entry points the data-parallel step needs, resolved at run time (dlopen of libnccl.so.2) so that the
// library carries no link-time dependency on NCCL; declarations follow nccl.h (ncclUniqueId is 128 opaque bytes passed
// by value, ncclFloat32 = 7, ncclSum = 0, ncclSuccess = 0).
struct NcclId { char internal[128]; };
struct NcclApi {
    void* lib = nullptr;
    int (*GetUniqueId)(NcclId*) = nullptr;
    int (*CommInitRank)(void**, int, NcclId, int) = nullptr;
    int (*CommDestroy)(void*) = nullptr;
    int (*AllReduce)(const void*, void*, size_t, int, int, void*, cudaStream_t) = nullptr;
    const char* (*GetErrorString)(int) = nullptr;
};
NcclApi* nccl_api(std::string* err) {
    static NcclApi api;
    static bool tried = false;
    if (!tried) {
        tried = true;
        void* h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
        if (!h) h = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
        if (h) {
            api.GetUniqueId = reinterpret_cast<int (*)(NcclId*)>(dlsym(h, "ncclGetUniqueId"));
            api.CommInitRank = reinterpret_cast<int (*)(void**, int, NcclId, int)>(dlsym(h, "ncclCommInitRank"));
            api.CommDestroy = reinterpret_cast<int (*)(void*)>(dlsym(h, "ncclCommDestroy"));
            api.AllReduce = reinterpret_cast<int (*)(const void*, void*, size_t, int, int, void*, cudaStream_t)>(dlsym(h, "ncclAllReduce"));
            api.GetErrorString = reinterpret_cast<const char* (*)(int)>(dlsym(h, "ncclGetErrorString"));
            if (api.GetUniqueId && api.CommInitRank && api.CommDestroy && api.AllReduce) api.lib = h;
        }
    }
    if (!api.lib) {
        if (err) *err = "NCCL is not available (libnccl.so.2 could not be loaded)";
        return nullptr;
    }
    return &api;
}

constexpr int kMaxBuckets = 8;
struct GradBucket {
    long long offset = 0, count = 0;
    int release_op = 0;  // the bucket's gradients are complete once backward has processed this op
};

struct ParamEntry {
    long long offset, size;
    int is_weight;   // decayed by l2 (conv filters, FC weights): Optimizers.cuh:27 isWeight
    int kind;        // 0 conv filter, 1 BN gamma, 2 BN beta, 3 FC weight, 4 FC bias
    int d0, d1, d2, d3;
};

}  // namespace

struct cbt_model {
    cb_ctx* ctx = nullptr;
    int batch = 0, classes = 0;
    std::vector<TensorBuf> t;
    std::vector<Op> ops;
    std::vector<ParamEntry> params;
    long long param_count = 0;
    float* P = nullptr;   // caller-owned flat buffers
    float* G = nullptr;
    float* M = nullptr;
    float* scratch = nullptr;      // one activation-sized temporary for accumulating data gradients
    long long scratch_elems = 0;
    float* labels = nullptr;       // device copy of the one-hot labels of the current step (caller-owned pointer)
    float* loss_dev = nullptr;     // device word: summed loss of the current step
    float* loss_n = nullptr;       // per-sample losses of the current step (fused head)
    int input = -1, logits = -1, probs = -1;
    std::vector<void*> owned;      // device allocations released by cbt_destroy
    std::string err;
    void* mom_table = nullptr;     // device descriptor table of the Momentum step, built by cbt_bind
    int bn_grad_swap = 0;          // 1: BatchNorm's two parameter gradients land in each other's slot, as in the reference
    int bn_groups = 1;             // BatchNorm statistics are taken per group of batch / bn_groups consecutive samples
    // data-parallel state (cbt_dp_init)
    void* comm = nullptr;
    int world = 1, rank = 0;
    cudaStream_t comm_stream = nullptr;
    cudaEvent_t bucket_ready[kMaxBuckets] = {};
    cudaEvent_t reduce_done = nullptr;
    std::vector<GradBucket> buckets;
    long long mom_biggest = 1;
    // weight-gradient streams (cbt_set_wgrad_streams): each has a context of its own (own scratch blocks) whose kernels
    // report into the main context's status word
    std::vector<cb_ctx*> side;
    std::vector<cudaStream_t> side_stream;
    std::vector<cudaEvent_t> side_fork, side_join;
    std::vector<int*> side_own_status;
    std::vector<char> side_used;
    int side_next = 0;
    // .crseq image of the model (ResNets): top-level operand ids, the words of the info section (uuid words flagged: a
    // file's own block numbering is accepted on load), and the parameter entries in the order the file stores them
    std::vector<uint32_t> crseq_ids, crseq_info;
    std::vector<uint8_t> crseq_info_is_uuid;
    std::vector<int> crseq_params;
};

extern "C" int cbt_set_wgrad_streams(cbt_model* m, int n);

namespace {

int new_tensor(cbt_model* m, int n, int c, int h, int w) {
    TensorBuf b;
    b.n = n; b.c = c; b.h = h; b.w = w;
    m->t.push_back(b);
    return (int)m->t.size() - 1;
}

long long add_param(cbt_model* m, long long size, int is_weight, int kind, int d0, int d1, int d2, int d3) {
    // keep every tensor 16-byte aligned inside the flat buffers (128-bit kernels, TMA bases)
    m->param_count = (m->param_count + 3) & ~3LL;
    ParamEntry e{m->param_count, size, is_weight, kind, d0, d1, d2, d3};
    m->params.push_back(e);
    m->param_count += size;
    return e.offset;
}

// channels [c_off, c_off + c) of tensor `parent` as a tensor of its own (no memory of its own)
int new_view(cbt_model* m, int parent, int c_off, int c) {
    const TensorBuf p = m->t[parent];
    const int id = new_tensor(m, p.n, c, p.h, p.w);
    m->t[id].view_of = parent;
    m->t[id].c_off = c_off;
    m->t[id].bstride = p.sample();
    return id;
}

// out >= 0: the result goes into that (view) tensor instead of a new one
int add_conv(cbt_model* m, int in, int oc, int f, int stride, int pad, int out = -1) {
    const TensorBuf& x = m->t[in];
    const int oh = (x.h - f + 2 * pad) / stride + 1, ow = (x.w - f + 2 * pad) / stride + 1;
    Op o{};
    o.kind = OP_CONV; o.in0 = in; o.oc = oc; o.f = f; o.stride = stride; o.pad = pad;
    o.w_off = add_param(m, (long long)oc * x.c * f * f, 1, 0, oc, x.c, f, f);
    o.out = out >= 0 ? out : new_tensor(m, x.n, oc, oh, ow);
    m->ops.push_back(o);
    return o.out;
}

// gamma_off / beta_off >= 0: parameters reserved earlier (the flat layout follows the reference's operand order, in
// which a block's second BatchNorm precedes its shortcut convolution, while the fused op must run after it)
int add_bn(cbt_model* m, int in, long long gamma_off = -1, long long beta_off = -1) {
    const TensorBuf x = m->t[in];
    Op o{};
    o.kind = OP_BN; o.in0 = in;
    const long long p = (long long)x.c * x.h * x.w;
    o.w_off = gamma_off >= 0 ? gamma_off : add_param(m, p, 0, 1, 1, x.c, x.h, x.w);   // gamma, shape (1,C,H,W): BatchNorm.cuh:27-33
    o.b_off = beta_off >= 0 ? beta_off : add_param(m, p, 0, 2, 1, x.c, x.h, x.w);     // beta
    // x-hat is only stored when the fused backward (which recomputes it from X) cannot serve this shape
    const bool fused = x.n <= 256 && (p % 4) == 0;
    o.xhat = fused ? -1 : new_tensor(m, x.n, x.c, x.h, x.w);
    o.out = new_tensor(m, x.n, x.c, x.h, x.w);
    m->ops.push_back(o);
    return o.out;
}

// BatchNorm followed by ReLU as one op when the fused kernels cover the shape (N <= 256, C*H*W % 4 == 0)
int add_relu(cbt_model* m, int in);
int add_bn_relu(cbt_model* m, int in) {
    const TensorBuf x = m->t[in];
    const long long p = (long long)x.c * x.h * x.w;
    if (!(x.n <= 256 && (p % 4) == 0)) return add_relu(m, add_bn(m, in));
    const int out = add_bn(m, in);
    m->ops.back().relu = true;
    return out;
}

// out = relu(BatchNorm(in) + shortcut): the end of a residual block as one op when the fused kernels cover the shape;
// otherwise BatchNorm, add-ReLU as separate ops
int add_add_relu(cbt_model* m, int a, int b);
int add_bn_add_relu(cbt_model* m, int in, int shortcut, long long gamma_off, long long beta_off) {
    const TensorBuf x = m->t[in];
    const long long p = (long long)x.c * x.h * x.w;
    if (!(x.n <= 256 && (p % 4) == 0)) return add_add_relu(m, add_bn(m, in, gamma_off, beta_off), shortcut);
    const int out = add_bn(m, in, gamma_off, beta_off);
    m->ops.back().relu = true;
    m->ops.back().in1 = shortcut;
    return out;
}

int add_relu(cbt_model* m, int in) {
    const TensorBuf x = m->t[in];
    Op o{};
    o.kind = OP_RELU; o.in0 = in;
    o.out = new_tensor(m, x.n, x.c, x.h, x.w);
    m->ops.push_back(o);
    return o.out;
}

int add_add(cbt_model* m, int a, int b) {
    const TensorBuf x = m->t[a];
    Op o{};
    o.kind = OP_ADD; o.in0 = a; o.in1 = b;
    o.out = new_tensor(m, x.n, x.c, x.h, x.w);
    m->ops.push_back(o);
    return o.out;
}

// out = relu(a + b): the shortcut add and the ReLU after it (archive/Resnet56:14-15) as one op
int add_add_relu(cbt_model* m, int a, int b) {
    const int out = add_add(m, a, b);
    m->ops.back().relu = true;
    return out;
}

// channel concatenation [in0 ; in1] (seblas concat, seblas/operations/cuConcat.cu:9-60, as ChannelConcatenater uses it)
int add_concat(cbt_model* m, int a, int b) {
    const TensorBuf x = m->t[a];
    const TensorBuf y = m->t[b];
    Op o{};
    o.kind = OP_CONCAT; o.in0 = a; o.in1 = b;
    o.out = new_tensor(m, x.n, x.c + y.c, x.h, x.w);
    m->ops.push_back(o);
    return o.out;
}

int add_avgpool2(cbt_model* m, int in, int out = -1) {
    const TensorBuf x = m->t[in];
    Op o{};
    o.kind = OP_AVGPOOL; o.in0 = in;
    o.out = out >= 0 ? out : new_tensor(m, x.n, x.c, x.h / 2, x.w / 2);
    m->ops.push_back(o);
    return o.out;
}

int add_gap(cbt_model* m, int in) {
    const TensorBuf x = m->t[in];
    Op o{};
    o.kind = OP_GAP; o.in0 = in;
    o.out = new_tensor(m, x.n, x.c, 1, 1);
    m->ops.push_back(o);
    return o.out;
}

int add_linear(cbt_model* m, int in, int out_features) {
    const TensorBuf x = m->t[in];
    const int in_features = x.c * x.h * x.w;
    Op o{};
    o.kind = OP_LINEAR; o.in0 = in; o.oc = out_features;
    o.w_off = add_param(m, (long long)out_features * in_features, 1, 3, out_features, in_features, 1, 1);
    o.b_off = add_param(m, out_features, 0, 4, out_features, 1, 1, 1);
    o.out = new_tensor(m, x.n, out_features, 1, 1);
    m->ops.push_back(o);
    return o.out;
}

int dev_alloc(cbt_model* m, float** p, long long elems) {
    void* q = nullptr;
    if (cudaMalloc(&q, (size_t)(elems > 0 ? elems : 1) * sizeof(float)) != cudaSuccess) {
        m->err = "cudaMalloc failed for an activation buffer";
        return CB_ENOMEM;
    }
    cudaMemset(q, 0, (size_t)(elems > 0 ? elems : 1) * sizeof(float));
    m->owned.push_back(q);
    *p = static_cast<float*>(q);
    return CB_OK;
}

// Head (global average pooling, dense layer, softmax cross-entropy), gradient-accumulation flags and buffers.
int finalize_model(cbt_model* m, int x, int classes) {
    const TensorBuf xin = m->t[x];
    if (classes <= 32 && xin.c <= 8192) {
        // one op: cb_head_fwd / cb_head_bwd
        Op o{};
        o.kind = OP_HEAD; o.in0 = x; o.oc = classes;
        o.w_off = add_param(m, (long long)classes * xin.c, 1, 3, classes, xin.c, 1, 1);
        o.b_off = add_param(m, classes, 0, 4, classes, 1, 1, 1);
        o.pooled = new_tensor(m, xin.n, xin.c, 1, 1);
        o.logits = new_tensor(m, xin.n, classes, 1, 1);
        o.probs = new_tensor(m, xin.n, classes, 1, 1);
        o.out = o.probs;
        m->logits = o.logits;
        m->probs = o.probs;
        m->ops.push_back(o);
    } else {
        x = add_gap(m, x);
        m->logits = add_linear(m, x, classes);
        Op o{};
        o.kind = OP_SOFTMAX_CE; o.in0 = m->logits;
        o.out = new_tensor(m, m->batch, classes, 1, 1);
        m->probs = o.out;
        m->ops.push_back(o);
    }
    m->param_count = (m->param_count + 3) & ~3LL;
    // in backward order the LAST forward consumer of a tensor writes its gradient first; every earlier consumer must
    // accumulate onto it
    // (views count as their parent: the gradient memory is shared, and the consumer of the widest view comes last in
    // the forward pass, so the first write in backward order covers every channel the later ones add to)
    auto root = [&](int id) { return m->t[id].view_of >= 0 ? m->t[id].view_of : id; };
    std::vector<int> seen(m->t.size(), 0);
    for (int i = (int)m->ops.size() - 1; i >= 0; --i) {
        Op& o = m->ops[i];
        if (o.in0 >= 0) {
            o.in0_grad_accumulate = seen[root(o.in0)] > 0;
            seen[root(o.in0)]++;
        }
        if (o.in1 >= 0) {
            o.in1_grad_accumulate = seen[root(o.in1)] > 0;
            seen[root(o.in1)]++;
        }
    }
    long long biggest = 0;
    for (size_t i = 0; i < m->t.size(); ++i) {
        TensorBuf& b = m->t[i];
        int rc = CB_OK;
        if ((int)i != m->input && b.view_of < 0) {  // the network input is read straight from the caller's batch buffer
            rc = dev_alloc(m, &b.a, b.size());
            if (rc == CB_OK) rc = dev_alloc(m, &b.d, b.size());
        }
        if (rc != CB_OK) return rc;
        if (b.size() > biggest) biggest = b.size();
    }
    for (TensorBuf& b : m->t) {
        if (b.view_of < 0) continue;
        const TensorBuf& par = m->t[(size_t)b.view_of];
        b.a = par.a + (long long)b.c_off * b.h * b.w;
        b.d = par.d + (long long)b.c_off * b.h * b.w;
    }
    m->scratch_elems = biggest;
    int rc = dev_alloc(m, &m->scratch, biggest);
    if (rc == CB_OK) rc = dev_alloc(m, &m->loss_dev, 4);
    if (rc == CB_OK) rc = dev_alloc(m, &m->loss_n, m->batch);
    if (rc == CB_OK) {
        const char* env = std::getenv("CBT_WGRAD_STREAMS");
        int n = env ? std::atoi(env) : 2;
        n = n < 0 ? 0 : (n > 4 ? 4 : n);
        rc = cbt_set_wgrad_streams(m, n);
    }
    return rc;
}

void release_side_streams(cbt_model* m) {
    for (size_t s = 0; s < m->side.size(); ++s) {
        cudaStreamSynchronize(m->side_stream[s]);
        m->side[s]->d_status = m->side_own_status[s];
        m->side[s]->stream = nullptr;
        cb_destroy(m->side[s]);
        cudaEventDestroy(m->side_fork[s]);
        cudaEventDestroy(m->side_join[s]);
        cudaStreamDestroy(m->side_stream[s]);
    }
    m->side.clear(); m->side_stream.clear(); m->side_fork.clear(); m->side_join.clear(); m->side_own_status.clear();
    m->side_used.clear();
}

#define CBT_TRY(expr)                                              \
    do {                                                           \
        int rc__ = (expr);                                         \
        if (rc__ != CB_OK) {                                       \
            m->err = cb_last_error(m->ctx);                        \
            return rc__;                                           \
        }                                                          \
    } while (0)

}  // namespace

extern "C" {

// ResNet of 6*blocks_per_stage + 2 layers on image_hw x image_hw RGB inputs (blocks_per_stage = 9: ResNet-56),
// channel plan 16/32/64, global average pooling and a `classes`-way dense head.
int cbt_resnet_create(cbt_model** out, cb_ctx* ctx, int batch, int blocks_per_stage, int image_hw, int classes) {
    if (!out || !ctx || batch < 1 || blocks_per_stage < 1 || image_hw < 4 || classes < 1) return CB_EINVAL;
    cbt_model* m = new cbt_model();
    m->ctx = ctx; m->batch = batch; m->classes = classes;
    cb_conv_cache_filters(ctx, 1);  // packed filters live from one weight update to the next
    int x = new_tensor(m, batch, 3, image_hw, image_hw);
    m->input = x;
    // the same network as the reference's operand list (archive/Resnet56: cuConv2D, BatchNorm, ReLU, then per block
    // ShortcutEndpoint begin, cuConv2D, BatchNorm, ReLU, cuConv2D, BatchNorm, ShortcutEndpoint end [1x1 cuConv2D], ReLU;
    // GlobalAvgPool, Linear, Softmax), recorded for the .crseq reader / writer as the model is built
    auto info_word = [&](uint32_t v, bool is_uuid = false) {
        m->crseq_info.push_back(v);
        m->crseq_info_is_uuid.push_back(is_uuid ? 1 : 0);
    };
    auto conv_info = [&](int oc_, int ic_, int f_, int stride_, int pad_) {
        for (uint32_t v : {(uint32_t)oc_, (uint32_t)ic_, (uint32_t)f_, (uint32_t)f_, (uint32_t)stride_, (uint32_t)stride_,
                           (uint32_t)pad_, (uint32_t)pad_, 0u})
            info_word(v);
    };
    auto last_entry = [&]() { return (int)m->params.size() - 1; };
    auto bn_entries = [&]() {  // the file stores beta before gamma (BatchNorm.cu:50-55)
        m->crseq_params.push_back(last_entry());
        m->crseq_params.push_back(last_entry() - 1);
    };
    x = add_conv(m, x, 16, 3, 1, 1);
    m->crseq_ids = {0xd002u, 0x0003u, 0xa002u};
    conv_info(16, 3, 3, 1, 1);
    m->crseq_params.push_back(last_entry());
    x = add_bn_relu(m, x);
    bn_entries();
    int ch = 16;
    uint32_t uuid = 1;
    for (int stage = 0; stage < 3; ++stage) {
        const int oc = 16 << stage;
        for (int b = 0; b < blocks_per_stage; ++b) {
            const int stride = (stage > 0 && b == 0) ? 2 : 1;
            for (uint32_t id : {0xf002u, 0xd002u, 0x0003u, 0xa002u, 0xd002u, 0x0003u, 0xf003u, 0xa002u}) m->crseq_ids.push_back(id);
            info_word(uuid, true);
            info_word(0);
            int y = add_conv(m, x, oc, 3, stride, 1);
            conv_info(oc, ch, 3, stride, 1);
            m->crseq_params.push_back(last_entry());
            y = add_bn_relu(m, y);
            bn_entries();
            y = add_conv(m, y, oc, 3, 1, 1);
            conv_info(oc, oc, 3, 1, 1);
            m->crseq_params.push_back(last_entry());
            const TensorBuf ty = m->t[y];
            const long long bn_p = (long long)ty.c * ty.h * ty.w;
            const long long g_off = add_param(m, bn_p, 0, 1, 1, ty.c, ty.h, ty.w);
            const long long b_off = add_param(m, bn_p, 0, 2, 1, ty.c, ty.h, ty.w);
            bn_entries();
            int sc = x;
            const bool projection = stride != 1 || ch != oc;
            info_word(uuid, true);
            info_word(projection ? 1 : 0);
            if (projection) {
                sc = add_conv(m, x, oc, 1, stride, 0);  // bare 1x1 projection
                info_word(0xd002u);
                conv_info(oc, ch, 1, stride, 0);
                m->crseq_params.push_back(last_entry());
            }
            x = add_bn_add_relu(m, y, sc, g_off, b_off);
            ch = oc;
            ++uuid;
        }
    }
    *out = m;
    const int rc = finalize_model(m, x, classes);
    for (uint32_t id : {0xb002u, 0x0001u, 0x0005u}) m->crseq_ids.push_back(id);
    info_word((uint32_t)classes);
    m->crseq_params.push_back(last_entry() - 1);  // Linear: weights, then biases
    m->crseq_params.push_back(last_entry());
    return rc;
}

// DenseNet-BC (growth k, `layers` bottleneck layers per dense block, compression 0.5): stem 3x3 conv to 2k, three dense
// blocks of [BN-ReLU-1x1 conv to 4k-BN-ReLU-3x3 conv to k, concatenated with the block input], transitions
// BN-ReLU-1x1 conv-2x2 average pooling, then BN-ReLU-global average pooling-dense head (layers = 16, k = 12:
// DenseNet-BC-100). Built from the reference's operand vocabulary (seann/operands/prefabs/DenseBlock.cuh:36-65).
int cbt_densenet_create(cbt_model** out, cb_ctx* ctx, int batch, int growth, int layers, int image_hw, int classes) {
    if (!out || !ctx || batch < 1 || growth < 1 || layers < 1 || image_hw < 8 || (image_hw & 3) || classes < 1) return CB_EINVAL;
    cbt_model* m = new cbt_model();
    m->ctx = ctx; m->batch = batch; m->classes = classes;
    cb_conv_cache_filters(ctx, 1);
    int x = new_tensor(m, batch, 3, image_hw, image_hw);
    m->input = x;
    // Every dense block is ONE buffer of all the channels it will ever hold; each layer reads the channel prefix that
    // exists so far (a view) and its 3x3 convolution writes the next `growth` channels in place, so the concatenation
    // [x ; y] the reference performs with a copy per layer (ChannelConcatenater over seblas::concat,
    // seblas/operations/cuConcat.cu:9-60) costs nothing here. The producer of a block's first channels (the stem, or
    // the pooling of the transition before it) writes into the buffer directly as well.
    int ch = 2 * growth, hw = image_hw;
    int block_buf = new_tensor(m, batch, ch + layers * growth, hw, hw);
    x = add_conv(m, x, ch, 3, 1, 1, new_view(m, block_buf, 0, ch));
    for (int block = 0; block < 3; ++block) {
        for (int l = 0; l < layers; ++l) {
            int y = add_conv(m, add_bn_relu(m, x), 4 * growth, 1, 1, 0);
            add_conv(m, add_bn_relu(m, y), growth, 3, 1, 1, new_view(m, block_buf, ch, growth));
            ch += growth;
            x = new_view(m, block_buf, 0, ch);  // for the last layer: the whole buffer
        }
        if (block < 2) {
            const int t = add_conv(m, add_bn_relu(m, x), ch / 2, 1, 1, 0);
            ch /= 2;
            hw /= 2;
            block_buf = new_tensor(m, batch, ch + layers * growth, hw, hw);
            x = add_avgpool2(m, t, new_view(m, block_buf, 0, ch));
        }
    }
    x = add_bn_relu(m, x);
    *out = m;
    return finalize_model(m, x, classes);
}

// The convolution weight gradients of the backward pass run on `n` streams of their own (0..4; 0 = on the context's
// stream like everything else). They are off the critical path of the backward pass (only the update needs them), so
// they fill the SMs the chain of data-gradient and BatchNorm kernels leaves idle. Each stream forks from the context's
// stream where the layer's output gradient is complete and joins it again at the end of cbt_backward. Not while the
// stream is being captured. New models start with the value of the environment variable CBT_WGRAD_STREAMS (default 2).
int cbt_set_wgrad_streams(cbt_model* m, int n) {
    if (!m || n < 0 || n > 4) return CB_EINVAL;
    cudaStreamSynchronize(m->ctx->stream);
    release_side_streams(m);
    for (int s = 0; s < n; ++s) {
        cudaStream_t st = nullptr;
        cudaEvent_t ef = nullptr, ej = nullptr;
        cb_ctx* c = nullptr;
        cudaError_t e = cudaStreamCreateWithFlags(&st, cudaStreamNonBlocking);
        if (e == cudaSuccess) e = cudaEventCreateWithFlags(&ef, cudaEventDisableTiming);
        if (e == cudaSuccess) e = cudaEventCreateWithFlags(&ej, cudaEventDisableTiming);
        if (e != cudaSuccess || cb_create(&c, m->ctx->device, st) != CB_OK) {
            m->err = "creating a weight-gradient stream failed";
            if (ef) cudaEventDestroy(ef);
            if (ej) cudaEventDestroy(ej);
            if (st) cudaStreamDestroy(st);
            release_side_streams(m);
            return CB_ECUDA;
        }
        m->side_own_status.push_back(c->d_status);
        c->d_status = m->ctx->d_status;
        // half the SMs per weight-gradient kernel: it shares the GPU with the data-gradient chain and with the other
        // weight-gradient streams, and fewer CTAs mean fewer partial sums to write and add (measured on the
        // ResNet-56 step: 74 CTAs beat 148, 49 and 37 at batch 128, and tie at batch 16)
        c->wgrad_grid_cap = m->ctx->sm_count / 2;
        m->side.push_back(c); m->side_stream.push_back(st); m->side_fork.push_back(ef); m->side_join.push_back(ej);
    }
    m->side_used.assign((size_t)n, 0);
    return CB_OK;
}

// Kernel launches made so far on the weight-gradient streams (the context's own counter does not see them).
long long cbt_side_launches(const cbt_model* m) {
    long long n = 0;
    if (m)
        for (const cb_ctx* c : m->side) n += c->launches;
    return n;
}

int cbt_destroy(cbt_model* m) {
    if (!m) return CB_EINVAL;
    cudaStreamSynchronize(m->ctx->stream);
    release_side_streams(m);
    for (void* p : m->owned) cudaFree(p);
    if (m->mom_table) cudaFree(m->mom_table);
    if (m->comm) {
        cudaStreamSynchronize(m->comm_stream);
        if (NcclApi* api = nccl_api(nullptr)) api->CommDestroy(m->comm);
        for (cudaEvent_t ev : m->bucket_ready)
            if (ev) cudaEventDestroy(ev);
        if (m->reduce_done) cudaEventDestroy(m->reduce_done);
        cudaStreamDestroy(m->comm_stream);
    }
    delete m;
    return CB_OK;
}

const char* cbt_last_error(const cbt_model* m) { return m ? m->err.c_str() : "null model"; }
long long cbt_param_count(const cbt_model* m) { return m ? m->param_count : 0; }
int cbt_param_entries(const cbt_model* m) { return m ? (int)m->params.size() : 0; }
// entry i: offset, size, is_weight, kind (0 conv filter, 1 BN gamma, 2 BN beta, 3 FC weight, 4 FC bias), dims[4]
int cbt_param_entry(const cbt_model* m, int i, long long* offset, long long* size, int* is_weight, int* kind, int* dims) {
    if (!m || i < 0 || i >= (int)m->params.size()) return CB_EINVAL;
    const ParamEntry& e = m->params[i];
    *offset = e.offset; *size = e.size; *is_weight = e.is_weight; *kind = e.kind;
    dims[0] = e.d0; dims[1] = e.d1; dims[2] = e.d2; dims[3] = e.d3;
    return CB_OK;
}
int cbt_op_count(const cbt_model* m) { return m ? (int)m->ops.size() : 0; }

// Binds the three caller-owned flat device buffers (each cbt_param_count floats, 16-byte aligned).
int cbt_bind(cbt_model* m, float* params, float* grads, float* momentum) {
    if (!m || !params || !grads || !momentum) return CB_EINVAL;
    if ((reinterpret_cast<uintptr_t>(params) | reinterpret_cast<uintptr_t>(grads) | reinterpret_cast<uintptr_t>(momentum)) & 15u) {
        m->err = "flat parameter buffers must be 16-byte aligned";
        return CB_EINVAL;
    }
    m->P = params; m->G = grads; m->M = momentum;
    const int n = (int)m->params.size();
    std::vector<float*> w(n), g(n), mo(n);
    std::vector<long long> sz(n);
    std::vector<unsigned char> fl(n);
    for (int i = 0; i < n; ++i) {
        const ParamEntry& e = m->params[i];
        w[i] = m->P + e.offset; g[i] = m->G + e.offset; mo[i] = m->M + e.offset;
        sz[i] = e.size; fl[i] = (unsigned char)e.is_weight;
    }
    if (m->mom_table) cudaFree(m->mom_table);
    m->mom_table = nullptr;
    int rc = cb::momentum_table_build(m->ctx, n, w.data(), g.data(), mo.data(), sz.data(), fl.data(), &m->mom_table,
                                      &m->mom_biggest);
    if (rc != CB_OK) m->err = cb_last_error(m->ctx);
    return rc;
}

// The caller wrote to the bound parameter buffer by a route of its own (initialisation, a checkpoint, a broadcast):
// packed copies of the filters are re-made before the next forward pass.
int cbt_params_changed(cbt_model* m) {
    if (!m) return CB_EINVAL;
    CBT_TRY(cb_filters_changed(m->ctx));
    return CB_OK;
}

// Writes the bound parameters as a .crseq file the reference's loadSequence reads (seio/modelcache/codec.cu:8-39 is the
// writer this mirrors; the file is replaced, where the reference appends to an existing one). ResNet models only.
int cbt_save_crseq(cbt_model* m, const char* path, unsigned epoch) {
    if (!m || !path || !m->P) return CB_EINVAL;
    if (m->crseq_ids.empty()) {
        m->err = "no .crseq image is defined for this model family";
        return CB_EUNSUPPORTED;
    }
    std::vector<float> host((size_t)m->param_count);
    if (cudaStreamSynchronize(m->ctx->stream) != cudaSuccess ||
        cudaMemcpy(host.data(), m->P, host.size() * sizeof(float), cudaMemcpyDeviceToHost) != cudaSuccess) {
        m->err = "reading the parameters back failed";
        return CB_ECUDA;
    }
    FILE* f = std::fopen(path, "wb");
    if (!f) {
        m->err = std::string("cannot open ") + path + " for writing";
        return CB_EINVAL;
    }
    const uint32_t head[3] = {0x7921aedfu, (uint32_t)m->crseq_ids.size(), (uint32_t)epoch};
    bool ok = std::fwrite(head, 4, 3, f) == 3;
    ok = ok && std::fwrite(m->crseq_ids.data(), 4, m->crseq_ids.size(), f) == m->crseq_ids.size();
    ok = ok && std::fwrite(m->crseq_info.data(), 4, m->crseq_info.size(), f) == m->crseq_info.size();
    for (int e : m->crseq_params) {
        const ParamEntry& pe = m->params[(size_t)e];
        ok = ok && std::fwrite(host.data() + pe.offset, 4, (size_t)pe.size, f) == (size_t)pe.size;
    }
    ok = (std::fclose(f) == 0) && ok;
    if (!ok) {
        m->err = std::string("writing ") + path + " failed";
        return CB_EINVAL;
    }
    return CB_OK;
}

// Loads the parameters of a .crseq file written by the reference's saveSequence (or by cbt_save_crseq) into the bound
// parameter buffer. The file's operand list and every geometry word must describe this model (block uuids are free);
// anything else is refused with the first difference named. *epoch receives the file's epoch id.
int cbt_load_crseq(cbt_model* m, const char* path, unsigned* epoch) {
    if (!m || !path || !m->P) return CB_EINVAL;
    if (m->crseq_ids.empty()) {
        m->err = "no .crseq image is defined for this model family";
        return CB_EUNSUPPORTED;
    }
    std::vector<uint8_t> bytes;
    {
        FILE* f = std::fopen(path, "rb");
        if (!f) {
            m->err = std::string("cannot open ") + path;
            return CB_EINVAL;
        }
        std::fseek(f, 0, SEEK_END);
        const long len = std::ftell(f);
        std::fseek(f, 0, SEEK_SET);
        bytes.resize(len > 0 ? (size_t)len : 0);
        const bool ok = bytes.empty() || std::fread(bytes.data(), 1, bytes.size(), f) == bytes.size();
        std::fclose(f);
        if (!ok) {
            m->err = std::string("reading ") + path + " failed";
            return CB_EINVAL;
        }
    }
    cb::CrseqModel parsed;
    if (!cb::crseq_parse(bytes, parsed, m->err)) return CB_EINVAL;
    const size_t n_ids = m->crseq_ids.size(), n_info = m->crseq_info.size();
    const size_t info_begin = 12 + 4 * n_ids;
    uint32_t file_count = 0;
    std::memcpy(&file_count, bytes.data() + 4, 4);
    if (file_count != n_ids || parsed.params_begin != info_begin + 4 * n_info) {
        m->err = "the file describes another network (" + std::to_string(file_count) + " operands, model has " + std::to_string(n_ids) + ")";
        return CB_EINVAL;
    }
    for (size_t i = 0; i < n_ids + n_info; ++i) {
        uint32_t v = 0;
        std::memcpy(&v, bytes.data() + 12 + 4 * i, 4);
        const bool is_id = i < n_ids;
        const uint32_t want = is_id ? m->crseq_ids[i] : m->crseq_info[i - n_ids];
        if (!is_id && m->crseq_info_is_uuid[i - n_ids]) continue;
        if (v != want) {
            m->err = std::string("the file describes another network: ") + (is_id ? "operand id " : "info word ") +
                     std::to_string(is_id ? i : i - n_ids) + " is " + std::to_string(v) + ", the model has " + std::to_string(want);
            return CB_EINVAL;
        }
    }
    size_t total = 0;
    for (int e : m->crseq_params) total += (size_t)m->params[(size_t)e].size;
    if (total * 4 != parsed.param_bytes) {
        m->err = "the file holds " + std::to_string(parsed.param_bytes / 4) + " parameter floats, the model has " + std::to_string(total);
        return CB_EINVAL;
    }
    std::vector<float> host((size_t)m->param_count, 0.f);
    size_t pos = parsed.params_begin;
    for (int e : m->crseq_params) {
        const ParamEntry& pe = m->params[(size_t)e];
        std::memcpy(host.data() + pe.offset, bytes.data() + pos, (size_t)pe.size * 4);
        pos += (size_t)pe.size * 4;
    }
    if (cudaStreamSynchronize(m->ctx->stream) != cudaSuccess ||
        cudaMemcpy(m->P, host.data(), host.size() * sizeof(float), cudaMemcpyHostToDevice) != cudaSuccess) {
        m->err = "copying the parameters to the device failed";
        return CB_ECUDA;
    }
    if (epoch) *epoch = parsed.epoch;
    return cbt_params_changed(m);
}

// Forward pass on `images` (batch x 3 x H x W, device) with one-hot `labels` (batch x classes, device). The images are
// read in place (no copy): they must stay unchanged until cbt_backward has run. Leaves the softmax in the last tensor
// and the summed loss in the model's device loss word (after cbt_backward for models with the fused head).
int cbt_forward(cbt_model* m, const float* images, const float* labels) {
    if (!m || !m->P || !images || !labels) return CB_EINVAL;
    cb_ctx* ctx = m->ctx;
    m->t[m->input].a = const_cast<float*>(images);
    m->labels = const_cast<float*>(labels);
    cudaError_t e;
    for (const Op& o : m->ops) {
        const TensorBuf& x = m->t[o.in0];
        TensorBuf& y = m->t[o.out];
        switch (o.kind) {
            case OP_CONV:
                if (x.bstride || y.bstride) {
                    cb_epilogue ep{};
                    ep.x_batch_stride = x.bstride;
                    ep.y_batch_stride = y.bstride;
                    CBT_TRY(cb_conv_fwd_ex(ctx, m->P + o.w_off, x.a, y.a, x.n, x.c, x.h, x.w, o.oc, o.f, o.f, o.stride, o.stride,
                                           o.pad, o.pad, &ep));
                    break;
                }
                CBT_TRY(cb_conv_fwd(ctx, m->P + o.w_off, x.a, y.a, nullptr, x.n, x.c, x.h, x.w, o.oc, o.f, o.f, o.stride,
                                    o.stride, o.pad, o.pad, 0));
                break;
            case OP_BN:
                if (m->bn_groups > 1) {
                    // statistics per group of consecutive samples: what each GPU of a data-parallel run computes on its shard
                    const long long P = (long long)x.c * x.h * x.w;
                    const int ng = x.n / m->bn_groups;
                    if (o.xhat >= 0 || x.n % m->bn_groups) {
                        m->err = "BatchNorm groups need the fused kernels (N <= 256, C*H*W % 4 == 0) and a batch divisible by the group count";
                        return CB_EUNSUPPORTED;
                    }
                    for (int g = 0; g < m->bn_groups; ++g) {
                        const long long off = (long long)g * ng * P;
                        CBT_TRY(cb::bn_fwd_group(ctx, x.a + off, m->P + o.b_off, m->P + o.w_off,
                                                 o.in1 >= 0 ? m->t[o.in1].a + off : nullptr, y.a + off, o.relu ? 1 : 0, ng, P));
                    }
                    break;
                }
                if (o.in1 >= 0) {
                    CBT_TRY(cb_bn_fwd_add_relu(ctx, x.a, m->P + o.b_off, m->P + o.w_off, m->t[o.in1].a, y.a, x.n,
                                               (long long)x.c * x.h * x.w));
                    break;
                }
                if (o.relu) {
                    CBT_TRY(cb_bn_fwd_relu_ex(ctx, x.a, m->P + o.b_off, m->P + o.w_off, y.a, x.n, (long long)x.c * x.h * x.w,
                                              x.bstride));
                    break;
                }
                if (x.bstride) {
                    m->err = "a BatchNorm without ReLU cannot read a view";
                    return CB_EUNSUPPORTED;
                }
                CBT_TRY(cb_bn_fwd(ctx, x.a, m->P + o.b_off, m->P + o.w_off, nullptr, nullptr, y.a,
                                  o.xhat >= 0 ? m->t[o.xhat].a : nullptr, x.n, (long long)x.c * x.h * x.w));
                break;
            case OP_RELU: CBT_TRY(cb_relu(ctx, x.a, y.a, x.size())); break;
            case OP_ADD: {
                // y = in0 + in1 (ShortcutEndpoint::forward, seann/operands/controlling/ShortcutEndpoint.cu:57-74)
                if (o.relu) {
                    CBT_TRY(cb_add_relu(ctx, x.a, m->t[o.in1].a, y.a, y.size()));
                    break;
                }
                e = cudaMemcpyAsync(y.a, x.a, (size_t)x.size() * 4, cudaMemcpyDeviceToDevice, ctx->stream);
                if (e != cudaSuccess) { m->err = cudaGetErrorString(e); return CB_ECUDA; }
                CBT_TRY(cb_tensor_op(ctx, CB_OP_ADD, y.a, m->t[o.in1].a, 0.f, y.size()));
                break;
            }
            case OP_CONCAT: {
                const TensorBuf& x1 = m->t[o.in1];
                const float* src[2] = {x.a, x1.a};
                const int ch[2] = {x.c, x1.c};
                CBT_TRY(cb_concat_channels(ctx, 2, src, ch, y.a, x.n, x.h * x.w));
                break;
            }
            case OP_AVGPOOL: CBT_TRY(cb_avgpool_ex(ctx, x.a, y.a, x.n, x.c, x.h, x.w, 2, 2, y.bstride)); break;
            case OP_GAP: CBT_TRY(cb_global_avgpool(ctx, x.a, y.a, (long long)x.n * x.c, x.h * x.w)); break;
            case OP_LINEAR:
                CBT_TRY(cb_linear_fwd(ctx, x.a, m->P + o.w_off, m->P + o.b_off, y.a, x.n, x.c * x.h * x.w, o.oc));
                break;
            case OP_SOFTMAX_CE:
                CBT_TRY(cb_softmax(ctx, x.a, y.a, x.n, x.c));
                CBT_TRY(cb_cross_entropy(ctx, y.a, labels, m->t[o.in0].d, m->loss_dev, y.size()));
                break;
            case OP_HEAD:
                CBT_TRY(cb_head_fwd(ctx, x.a, m->P + o.w_off, m->P + o.b_off, labels, m->t[o.pooled].a, m->t[o.logits].a,
                                    m->t[o.probs].a, m->t[o.logits].d, m->loss_n, x.n, x.c, x.h * x.w, o.oc));
                break;
        }
    }
    return CB_OK;
}

// Data-parallel gradient exchange: every bucket (a contiguous range of the flat gradient buffer) whose last parameter
// gradient was produced by op `op_index` is sum-allreduced on the communication stream, which waits for the compute
// stream at that point only — the rest of the backward pass overlaps the transfer.
static int dp_release_buckets(cbt_model* m, int op_index) {
    NcclApi* api = nccl_api(&m->err);
    if (!api) return CB_EUNSUPPORTED;
    for (size_t b = 0; b < m->buckets.size(); ++b) {
        const GradBucket& bk = m->buckets[b];
        if (bk.release_op != op_index || bk.count == 0) continue;
        cudaError_t e = cudaEventRecord(m->bucket_ready[b], m->ctx->stream);
        if (e == cudaSuccess) e = cudaStreamWaitEvent(m->comm_stream, m->bucket_ready[b], 0);
        // weight gradients of the bucket may still be in flight on their own streams
        for (size_t s = 0; s < m->side.size() && e == cudaSuccess; ++s) {
            if (!m->side_used[s]) continue;
            e = cudaEventRecord(m->side_join[s], m->side_stream[s]);
            if (e == cudaSuccess) e = cudaStreamWaitEvent(m->comm_stream, m->side_join[s], 0);
        }
        if (e != cudaSuccess) { m->err = cudaGetErrorString(e); return CB_ECUDA; }
        const int rc = api->AllReduce(m->G + bk.offset, m->G + bk.offset, (size_t)bk.count, 7 /* ncclFloat32 */, 0 /* ncclSum */,
                                      m->comm, m->comm_stream);
        if (rc != 0) {
            m->err = std::string("ncclAllReduce: ") + (api->GetErrorString ? api->GetErrorString(rc) : "failed");
            return CB_ECUDA;
        }
    }
    return CB_OK;
}

// Backward pass: fills the flat gradient buffer (accumulating into it, as every seblas parameter-gradient kernel
// does; cbt_update zeroes it again).
int cbt_backward(cbt_model* m) {
    if (!m || !m->G) return CB_EINVAL;
    cb_ctx* ctx = m->ctx;
    m->side_next = 0;
    std::fill(m->side_used.begin(), m->side_used.end(), 0);
    for (int i = (int)m->ops.size() - 1; i >= 0; --i) {
        const Op& o = m->ops[i];
        TensorBuf& x = m->t[o.in0];
        TensorBuf& y = m->t[o.out];
        const bool to_input = o.in0 == m->input;  // the network input needs no gradient
        // Ops whose kernel can add onto an existing gradient write x.d directly; the others go through the scratch
        // buffer followed by x.d += scratch when an earlier consumer already wrote x.d.
        const bool bn_native = o.kind == OP_BN && o.xhat < 0 && o.in1 < 0 && m->bn_groups == 1;
        const bool native_acc = o.kind == OP_CONV || o.kind == OP_ADD || bn_native;
        if (x.bstride && !(o.kind == OP_CONV || bn_native)) {
            m->err = "only convolutions and fused BatchNorm-ReLU layers can read a view";
            return CB_EUNSUPPORTED;
        }
        float* dx = (o.in0_grad_accumulate && !native_acc) ? m->scratch : x.d;
        switch (o.kind) {
            case OP_SOFTMAX_CE: break;  // the forward already wrote softmax - labels into the logits' gradient
            case OP_HEAD:
                CBT_TRY(cb_head_bwd(ctx, m->t[o.logits].d, m->t[o.pooled].a, m->P + o.w_off, dx, m->G + o.w_off, m->G + o.b_off,
                                    m->loss_n, m->loss_dev, x.n, x.c, x.h * x.w, o.oc));
                break;
            case OP_LINEAR:
                CBT_TRY(cb_linear_paramgrad(ctx, y.d, x.a, m->G + o.w_off, m->G + o.b_off, x.n, x.c * x.h * x.w, o.oc));
                CBT_TRY(cb_linear_xgrad(ctx, y.d, m->P + o.w_off, dx, x.n, x.c * x.h * x.w, o.oc));
                break;
            case OP_CONCAT: {
                // split dY: the new features (in1) take their slice directly, the carried input (in0) its own
                TensorBuf& x1 = m->t[o.in1];
                const size_t pl = (size_t)x.h * x.w * 4;
                cudaError_t e = cudaMemcpy2DAsync(x1.d, (size_t)x1.c * pl, y.d + (size_t)x.c * x.h * x.w, (size_t)y.c * pl,
                                                  (size_t)x1.c * pl, x.n, cudaMemcpyDeviceToDevice, ctx->stream);
                if (e == cudaSuccess)
                    e = cudaMemcpy2DAsync(dx, (size_t)x.c * pl, y.d, (size_t)y.c * pl, (size_t)x.c * pl, x.n,
                                          cudaMemcpyDeviceToDevice, ctx->stream);
                if (e != cudaSuccess) { m->err = cudaGetErrorString(e); return CB_ECUDA; }
                break;
            }
            case OP_AVGPOOL: CBT_TRY(cb_avgpool_back_ex(ctx, dx, y.d, x.n, x.c, x.h, x.w, 2, 2, y.bstride)); break;
            case OP_GAP: CBT_TRY(cb_global_avgpool_back(ctx, dx, y.d, (long long)x.n * x.c, x.h * x.w)); break;
            case OP_RELU: CBT_TRY(cb_relu_grad(ctx, x.a, y.d, dx, x.size())); break;
            case OP_ADD: {
                // both inputs receive dY (ShortcutEndpoint::xGrads routes the same gradient to the skip path)
                TensorBuf& x1 = m->t[o.in1];
                if (o.relu && !o.in0_grad_accumulate && !o.in1_grad_accumulate) {
                    CBT_TRY(cb_relu_grad2(ctx, y.a, y.d, x.d, x1.d, y.size()));
                    continue;
                }
                if (o.relu) CBT_TRY(cb_relu_grad2(ctx, y.a, y.d, y.d, nullptr, y.size()));  // mask in place, then route
                for (int k = 0; k < 2; ++k) {
                    TensorBuf& t = k ? x1 : x;
                    const bool acc = k ? o.in1_grad_accumulate : o.in0_grad_accumulate;
                    if (acc) {
                        CBT_TRY(cb_tensor_op(ctx, CB_OP_ADD, t.d, y.d, 0.f, t.size()));
                    } else {
                        cudaError_t e = cudaMemcpyAsync(t.d, y.d, (size_t)y.size() * 4, cudaMemcpyDeviceToDevice, ctx->stream);
                        if (e != cudaSuccess) { m->err = cudaGetErrorString(e); return CB_ECUDA; }
                    }
                }
                continue;
            }
            case OP_BN: {
                // where d(gamma) and d(beta) are stored: their own slots, or each other's (reference order)
                float* dgamma = m->G + (m->bn_grad_swap ? o.b_off : o.w_off);
                float* dbeta = m->G + (m->bn_grad_swap ? o.w_off : o.b_off);
                const long long P = (long long)x.c * x.h * x.w;
                if (m->bn_groups > 1) {
                    if (x.bstride) {
                        m->err = "BatchNorm groups are not combined with views";
                        return CB_EUNSUPPORTED;
                    }
                    const int ng = x.n / m->bn_groups;
                    for (int g = 0; g < m->bn_groups; ++g) {
                        const long long off = (long long)g * ng * P;
                        CBT_TRY(cb::bn_bwd_group(ctx, y.d + off, m->P + o.w_off, x.a + off, dx + off, dgamma, dbeta,
                                                 o.relu ? y.a + off : nullptr, o.in1 >= 0 ? m->t[o.in1].d + off : nullptr,
                                                 o.in1_grad_accumulate ? 1 : 0, g > 0 ? 1 : 0, ng, P));
                    }
                } else if (o.in1 >= 0) {
                    CBT_TRY(cb_bn_bwd_fused_res(ctx, y.d, m->P + o.w_off, x.a, dx, dgamma, dbeta, y.a, m->t[o.in1].d,
                                                o.in1_grad_accumulate ? 1 : 0, x.n, P));
                } else if (o.xhat < 0) {
                    // (dx is x.d here: this form adds onto an existing gradient itself, also through a view's stride)
                    CBT_TRY(cb_bn_bwd_fused_ex(ctx, y.d, m->P + o.w_off, x.a, dx, dgamma, dbeta, o.relu ? y.a : nullptr, x.n, P,
                                               x.bstride, x.bstride, o.in0_grad_accumulate ? 1 : 0));
                } else {
                    CBT_TRY(cb_bn_paramgrad(ctx, y.d, m->t[o.xhat].a, dgamma, dbeta, x.n, P));
                    CBT_TRY(cb_bn_bwd(ctx, y.d, m->P + o.w_off, x.a, dx, x.n, P));
                }
                break;
            }
            case OP_CONV: {
                cb_ctx* wc = ctx;
                if (!m->side.empty()) {
                    // fork: the weight gradient needs this layer's output gradient (complete at this point of the
                    // context's stream) and its input, and nothing later in the backward pass needs the result
                    const size_t s = (size_t)(m->side_next++) % m->side.size();
                    wc = m->side[s];
                    wc->math = ctx->math;
                    wc->deterministic = ctx->deterministic;
                    wc->workspace_frozen = ctx->workspace_frozen;
                    cudaError_t e = cudaEventRecord(m->side_fork[s], ctx->stream);
                    if (e == cudaSuccess) e = cudaStreamWaitEvent(m->side_stream[s], m->side_fork[s], 0);
                    if (e != cudaSuccess) { m->err = cudaGetErrorString(e); return CB_ECUDA; }
                    m->side_used[s] = 1;
                }
                const int rc_w = cb_conv_wgrad_ex(wc, y.d, x.a, m->G + o.w_off, x.n, x.c, x.h, x.w, o.oc, o.f, o.f, o.stride,
                                                  o.stride, o.pad, o.pad, 1, y.bstride, x.bstride);
                if (rc_w != CB_OK) { m->err = cb_last_error(wc); return rc_w; }
                if (!to_input)
                    CBT_TRY(cb_conv_dgrad_ex(ctx, m->P + o.w_off, y.d, x.d, x.n, x.c, x.h, x.w, o.oc, o.f, o.f, o.stride,
                                             o.stride, o.pad, o.pad, o.in0_grad_accumulate ? 1 : 0, y.bstride, x.bstride));
                break;
            }
        }
        if (o.in0_grad_accumulate && !native_acc && !to_input)
            CBT_TRY(cb_tensor_op(ctx, CB_OP_ADD, x.d, m->scratch, 0.f, x.size()));
        if (m->comm) {
            int rc = dp_release_buckets(m, i);
            if (rc != CB_OK) return rc;
        }
    }
    // join: everything queued on the context's stream after this call sees every weight gradient
    for (size_t s = 0; s < m->side.size(); ++s) {
        if (!m->side_used[s]) continue;
        cudaError_t e = cudaEventRecord(m->side_join[s], m->side_stream[s]);
        if (e == cudaSuccess) e = cudaStreamWaitEvent(ctx->stream, m->side_join[s], 0);
        if (e != cudaSuccess) { m->err = cudaGetErrorString(e); return CB_ECUDA; }
    }
    if (m->comm) {
        // the gradients are summed over the ranks by the time anything later on the context's stream reads them
        cudaError_t e = cudaEventRecord(m->reduce_done, m->comm_stream);
        if (e == cudaSuccess) e = cudaStreamWaitEvent(ctx->stream, m->reduce_done, 0);
        if (e != cudaSuccess) { m->err = cudaGetErrorString(e); return CB_ECUDA; }
    }
    return CB_OK;
}

// The reference's BatchNorm operand hands beta's gradient tensor to the kernel argument that receives d(gamma) and
// gamma's to the one that receives d(beta) (seann/operands/seblas/BatchNorm.cu:24 against the parameter order of
// seblas/operations/cuBatchNorm.cuh:16), so its Momentum step moves beta by d(gamma) and gamma by d(beta). on = 1
// reproduces that order, for runs that must follow the reference's operand graph step by step; the default (0) is the
// mathematically right assignment.
int cbt_set_reference_bn_grad_order(cbt_model* m, int on) {
    if (!m) return CB_EINVAL;
    m->bn_grad_swap = on ? 1 : 0;
    return CB_OK;
}

// BatchNorm statistics per group of batch / groups consecutive samples (1 = the whole batch, the default). A run on
// one GPU with G groups computes exactly what G data-parallel ranks compute on their shards of the same batch, which
// is how the sharded step is validated against the oracle.
int cbt_set_bn_groups(cbt_model* m, int groups) {
    if (!m || groups < 1 || m->batch % groups) return CB_EINVAL;
    m->bn_groups = groups;
    return CB_OK;
}

// ---- data-parallel training: one process per GPU, each with its own model on its shard of the batch
// Rank 0 creates the 128-byte rendezvous id and sends it to the other ranks by any host-side channel.
int cbt_dp_unique_id(char* id128) {
    if (!id128) return CB_EINVAL;
    NcclApi* api = nccl_api(nullptr);
    if (!api) return CB_EUNSUPPORTED;
    NcclId id;
    if (api->GetUniqueId(&id) != 0) return CB_ECUDA;
    std::memcpy(id128, id.internal, 128);
    return CB_OK;
}

// Joins the communicator (collective over all ranks) and splits the flat gradient buffer into `buckets` ranges (1..8)
// that double in size from the first layers' end (1 : 2 : 4 ...). From then on cbt_backward sum-allreduces each range over the ranks on a communication
// stream as soon as its last gradient has been produced, and the gradients are the sums over all ranks when
// cbt_backward's work is done. Call before capturing the step in a CUDA graph.
int cbt_dp_init(cbt_model* m, const char* id128, int world, int rank, int buckets) {
    if (const char* e = std::getenv("CBT_DP_BUCKETS")) buckets = std::atoi(e);  // development override
    if (!m || !id128 || world < 1 || rank < 0 || rank >= world || buckets < 1 || buckets > kMaxBuckets) return CB_EINVAL;
    if (m->comm) return CB_EINVAL;
    NcclApi* api = nccl_api(&m->err);
    if (!api) return CB_EUNSUPPORTED;
    NcclId id;
    std::memcpy(id.internal, id128, 128);
    void* comm = nullptr;
    const int rc = api->CommInitRank(&comm, world, id, rank);
    if (rc != 0) {
        m->err = std::string("ncclCommInitRank: ") + (api->GetErrorString ? api->GetErrorString(rc) : "failed");
        return CB_ECUDA;
    }
    cudaError_t e = cudaStreamCreateWithFlags(&m->comm_stream, cudaStreamNonBlocking);
    for (int b = 0; b < buckets && e == cudaSuccess; ++b) e = cudaEventCreateWithFlags(&m->bucket_ready[b], cudaEventDisableTiming);
    if (e == cudaSuccess) e = cudaEventCreateWithFlags(&m->reduce_done, cudaEventDisableTiming);
    if (e != cudaSuccess) { m->err = cudaGetErrorString(e); return CB_ECUDA; }
    m->comm = comm; m->world = world; m->rank = rank;
    // bucket b covers parameter entries whose offsets fall in [lo_b, hi_b); it is released by the FIRST op (in forward
    // order) owning one of them, the last of them to be reached by the backward pass
    m->buckets.assign((size_t)buckets, GradBucket{});
    const long long total = m->param_count;
    // The bucket at the lowest offsets holds the first layers: it is released last and nothing is left to overlap its
    // exchange with, so the ranges double in size from there (1 : 2 : 4 ...) instead of being equal.
    const char* ge = std::getenv("CBT_DP_GEOMETRIC");  // development switch
    const bool geometric = ge ? std::atoi(ge) != 0 : true;
    const long long units = geometric ? (1LL << buckets) - 1 : buckets;
    for (int b = 0; b < buckets; ++b) {
        const long long u0 = geometric ? (1LL << b) - 1 : b, u1 = geometric ? (1LL << (b + 1)) - 1 : b + 1;
        long long lo = total * u0 / units, hi = total * u1 / units;
        lo &= ~3LL;
        hi = b + 1 == buckets ? total : (hi & ~3LL);
        m->buckets[b].offset = lo;
        m->buckets[b].count = hi - lo;
        m->buckets[b].release_op = (int)m->ops.size();
    }
    auto claim = [&](long long off, long long size, int op) {
        for (GradBucket& bk : m->buckets)
            if (off < bk.offset + bk.count && off + size > bk.offset && op < bk.release_op) bk.release_op = op;
    };
    for (int i = 0; i < (int)m->ops.size(); ++i) {
        const Op& o = m->ops[i];
        for (const ParamEntry& pe : m->params)
            if (pe.offset == o.w_off || pe.offset == o.b_off) claim(pe.offset, pe.size, i);
    }
    for (GradBucket& bk : m->buckets)
        if (bk.release_op >= (int)m->ops.size()) bk.release_op = 0;  // no parameters inside (padding only)
    return CB_OK;
}

int cbt_dp_world(const cbt_model* m) { return m ? m->world : 0; }

// One Momentum step over every parameter tensor (one launch). BN parameter gradients are assigned, not
// accumulated, by cb_bn_paramgrad, exactly like the reference kernel (cuBatchNorm.cu:128-147).
int cbt_update(cbt_model* m, float lr, float beta, float l2) {
    if (!m || !m->P || !m->mom_table) return CB_EINVAL;
    CBT_TRY(cb::momentum_table_launch(m->ctx, m->mom_table, (int)m->params.size(), m->mom_biggest, lr, beta, l2));
    return CB_OK;
}

// Mean loss per sample of the last forward pass (synchronises the stream).
int cbt_loss(cbt_model* m, float* loss_mean) {
    if (!m || !loss_mean) return CB_EINVAL;
    float s = 0.f;
    cudaError_t e = cudaStreamSynchronize(m->ctx->stream);
    if (e == cudaSuccess && !m->ops.empty() && m->ops.back().kind == OP_HEAD) {
        // fused head: the forward pass leaves one loss per sample; they are summed here in sample order
        std::vector<float> per((size_t)m->batch);
        e = cudaMemcpy(per.data(), m->loss_n, sizeof(float) * per.size(), cudaMemcpyDeviceToHost);
        for (float v : per) s += v;
    } else if (e == cudaSuccess) {
        e = cudaMemcpy(&s, m->loss_dev, sizeof(float), cudaMemcpyDeviceToHost);
    }
    if (e != cudaSuccess) { m->err = cudaGetErrorString(e); return CB_ECUDA; }
    *loss_mean = s / (float)m->batch;
    return CB_OK;
}

// Device pointers for tests: value (grad = 0) or gradient (grad = 1) of tensor `id`; -1 = logits, -2 = softmax.
float* cbt_tensor_ptr(cbt_model* m, int id, int grad) {
    if (!m) return nullptr;
    if (id == -1) id = m->logits;
    if (id == -2) id = m->probs;
    if (id < 0 || id >= (int)m->t.size()) return nullptr;
    return grad ? m->t[id].d : m->t[id].a;
}
float* cbt_loss_ptr(cbt_model* m) { return m ? m->loss_dev : nullptr; }
// Copies the summed loss word of the last step (written by the backward pass for models with the fused head) to a
// caller-owned device float, in stream order.
int cbt_copy_loss(cbt_model* m, float* dst) {
    if (!m || !dst) return CB_EINVAL;
    cudaError_t e = cudaMemcpyAsync(dst, m->loss_dev, sizeof(float), cudaMemcpyDeviceToDevice, m->ctx->stream);
    if (e != cudaSuccess) { m->err = cudaGetErrorString(e); return CB_ECUDA; }
    return CB_OK;
}
// Copies n floats of a tensor (see cbt_tensor_ptr) into the caller's device buffer, in stream order.
int cbt_copy_tensor(cbt_model* m, int id, int grad, float* dst, long long n) {
    float* src = cbt_tensor_ptr(m, id, grad);
    if (!src || !dst || n < 0) return CB_EINVAL;
    cudaError_t e = cudaMemcpyAsync(dst, src, (size_t)n * 4, cudaMemcpyDeviceToDevice, m->ctx->stream);
    if (e != cudaSuccess) { m->err = cudaGetErrorString(e); return CB_ECUDA; }
    return CB_OK;
}

}  // extern "C"
