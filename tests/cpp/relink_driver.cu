// Driver for the relink test: builds a ResNet-(6n+2) out of the REFERENCE's own operand classes (compiled from the
// reference tree by oracle/build_relink.sh against this library's header shim) and runs the reference's own
// Sequential::forward / backward / learn on it, so the training step of the reference's operand graph executes on the
// sm_100a kernels. The topology is the one of archive/Resnet56 (ShortcutEndpoint pairs around conv-BN-ReLU-conv-BN,
// a bare 1x1 stride-2 cuConv2D in the shortcut where the shape changes) with the GlobalAvgPool + Linear head.
//
//   relink_driver train <blocks> <batch> <hw> <classes> <steps> <math> <lr> <in.bin> <out.bin>
//       in.bin : flat parameters (layout below), images (batch*3*hw*hw), one-hot labels (batch*classes), fp32
//       out.bin: mean loss of every step (steps floats), parameters after the last step, gradients of step 1
//   relink_driver save  <blocks> <batch> <hw> <classes> <in.bin> <out.crseq>
//       writes the model with the reference's own codec (seio::saveSequence)
//   relink_driver loop  <batch> <hw>
//       random initialisation + the synthetic Dataset + the reference's Sequential::train for two batches
//
// Flat parameter layout (the training executor's): every tensor starts at a multiple of 4 floats; operands in order;
// cuConv2D: filter; BatchNorm: gamma, beta; ShortcutEndpoint(end): its branch convolution's filter; Linear: weights,
// biases. Gradients are written exactly as the operands hold them, i.e. with BatchNorm's two gradients in the slots
// the reference's BatchNorm::paramGrads puts them (seann/operands/seblas/BatchNorm.cu:24 passes beta's and gamma's
// gradient tensors in swapped order).
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>

#include "seann/seann.cuh"
#include "seio/modelcache/codec.cuh"

using namespace seann;
using namespace seblas;

namespace {

struct Slot {
    NetParam* p;
    size_t offset;
};

std::vector<float> readFile(const char* path) {
    FILE* f = std::fopen(path, "rb");
    if (!f) { std::fprintf(stderr, "cannot open %s\n", path); std::exit(2); }
    std::fseek(f, 0, SEEK_END);
    const long n = std::ftell(f);
    std::fseek(f, 0, SEEK_SET);
    std::vector<float> v((size_t)n / 4);
    if (std::fread(v.data(), 4, v.size(), f) != v.size()) { std::fprintf(stderr, "short read on %s\n", path); std::exit(2); }
    std::fclose(f);
    return v;
}

Sequential* buildResnet(int blocks, int batch, int hw, int classes, std::vector<OperandBase*>& ops) {
    ops.push_back(new cuConv2D(shape4(16, 3, 3, 3), 1, 1, 1, 1, false));
    ops.push_back(new BatchNorm());
    ops.push_back(new ReLU());
    uint32 uuid = 1;
    int ch = 16;
    for (int stage = 0; stage < 3; ++stage) {
        const int oc = 16 << stage;
        for (int b = 0; b < blocks; ++b, ++uuid) {
            const uint32 stride = (stage > 0 && b == 0) ? 2 : 1;
            ops.push_back(new ShortcutEndpoint(false, uuid, {}));
            ops.push_back(new cuConv2D(shape4(oc, ch, 3, 3), stride, stride, 1, 1, false));
            ops.push_back(new BatchNorm());
            ops.push_back(new ReLU());
            ops.push_back(new cuConv2D(shape4(oc, oc, 3, 3), 1, 1, 1, 1, false));
            ops.push_back(new BatchNorm());
            if (stride != 1 || ch != oc)
                ops.push_back(new ShortcutEndpoint(true, uuid, {new cuConv2D(shape4(oc, ch, 1, 1), stride, stride, 0, 0, false)}));
            else
                ops.push_back(new ShortcutEndpoint(true, uuid, {}));
            ops.push_back(new ReLU());
            ch = oc;
        }
    }
    ops.push_back(new GlobalAvgPool());
    ops.push_back(new Linear(classes));
    ops.push_back(new Softmax());
    OperandBase** arr;
    cudaMallocHost(&arr, sizeof(OperandBase*) * ops.size());
    for (size_t i = 0; i < ops.size(); ++i) arr[i] = ops[i];
    return new Sequential(shape4(batch, 3, hw, hw), (uint32)ops.size(), arr);
}

size_t collectSlots(const std::vector<OperandBase*>& ops, std::vector<Slot>& slots) {
    size_t off = 0;
    auto add = [&](NetParam* p) {
        off = (off + 3) & ~size_t(3);
        slots.push_back({p, off});
        off += p->data()->dims.size;
    };
    for (OperandBase* o : ops) {
        switch (o->OPERAND_ID()) {
            case OPR_CUDNN_CONV2D: add(((cuConv2D*)o)->filter); break;
            case OPR_SEBLAS_BATCHNORM: add(((BatchNorm*)o)->gamma); add(((BatchNorm*)o)->beta); break;
            case OPR_CTRL_SHORTCUTENDPOINT_END: {
                auto* s = (ShortcutEndpoint*)o;
                for (uint32 i = 0; i < s->operandCount; ++i) add(((cuConv2D*)s->branchOperands[i])->filter);
                break;
            }
            case OPR_SEBLAS_LINEAR: add(((Linear*)o)->weights); add(((Linear*)o)->biases); break;
            default: break;
        }
    }
    return (off + 3) & ~size_t(3);
}

int mathMode(const char* s) {
    if (!std::strcmp(s, "tf32")) return CB_MATH_TF32;
    if (!std::strcmp(s, "3xtf32")) return CB_MATH_3XTF32;
    if (!std::strcmp(s, "fp32")) return CB_MATH_FP32;
    std::fprintf(stderr, "unknown math mode %s\n", s);
    std::exit(2);
}

void loadParams(const std::vector<Slot>& slots, const float* flat) {
    for (const Slot& s : slots)
        cudaMemcpy(s.p->data()->elements, flat + s.offset, sizeof(float) * s.p->data()->dims.size, cudaMemcpyHostToDevice);
}

}  // namespace

int main(int argc, char** argv) {
    try {
        if (argc >= 2 && !std::strcmp(argv[1], "loop")) {
            const int batch = std::atoi(argv[2]), hw = std::atoi(argv[3]);
            std::vector<OperandBase*> ops;
            Sequential* model = buildResnet(1, batch, hw, 10, ops);
            model->construct(new OPTIMIZER_MOMENTUM(0.01f / batch));
            seblas::setRandSeed(7);
            model->randInit();
            model->setLoss(crossEntropyLoss, crossEntropyCalc);
            // one epoch of three batches' worth of samples: the loop trains on two batches, then the loader reports the
            // next epoch and the loop ends (after writing its .crseq cache file into the working directory)
            auto* data = seio::Dataset::construct(batch, batch, 3 * batch, 1, shape4(3, hw, hw), shape4(10, 1));
            model->train(data, false, 1);
            std::printf("relink loop ok: %u batches drawn, last batch loss %f\n", data->batchID, data->procDisplay->epochTrainLoss);
            return 0;
        }
        if (argc < 8) { std::fprintf(stderr, "usage: see the header of tests/cpp/relink_driver.cu\n"); return 2; }
        const bool save = !std::strcmp(argv[1], "save");
        const int blocks = std::atoi(argv[2]), batch = std::atoi(argv[3]), hw = std::atoi(argv[4]), classes = std::atoi(argv[5]);
        std::vector<OperandBase*> ops;
        Sequential* model = buildResnet(blocks, batch, hw, classes, ops);
        if (save) {
            model->construct(new OPTIMIZER_MOMENTUM(0.01f));
            std::vector<Slot> slots;
            const size_t total = collectSlots(ops, slots);
            std::vector<float> in = readFile(argv[6]);
            if (in.size() < total) { std::fprintf(stderr, "input file too short\n"); return 2; }
            loadParams(slots, in.data());
            std::remove(argv[7]);
            seio::saveSequence(argv[7], model, 3);
            std::printf("relink save ok: %zu operands, %zu parameter floats\n", ops.size(), total);
            return 0;
        }
        if (argc < 11) { std::fprintf(stderr, "usage: see the header of tests/cpp/relink_driver.cu\n"); return 2; }
        const int steps = std::atoi(argv[6]);
        const float lr = (float)std::atof(argv[8]);
        model->construct(new OPTIMIZER_MOMENTUM(lr));
        seblas::setMathMode(mathMode(argv[7]));
        model->setLoss(crossEntropyLoss, crossEntropyCalc);
        std::vector<Slot> slots;
        const size_t total = collectSlots(ops, slots);
        std::vector<float> in = readFile(argv[9]);
        const size_t nimg = (size_t)batch * 3 * hw * hw, nlab = (size_t)batch * classes;
        if (in.size() != total + nimg + nlab) {
            std::fprintf(stderr, "input file holds %zu floats, expected %zu + %zu + %zu\n", in.size(), total, nimg, nlab);
            return 2;
        }
        loadParams(slots, in.data());
        Tensor* X = Tensor::declare(batch, 3, hw, hw)->ripOffHost(in.data() + total);
        Tensor* label = Tensor::declare(batch, 1, classes, 1)->ripOffHost(in.data() + total + nimg);
        Tensor* lossBuf = Tensor::create(model->netY->A->dims);
        std::vector<float> losses((size_t)steps), grads(total, 0.f), params(total, 0.f);
        for (int s = 0; s < steps; ++s) {
            // the body of the reference's training loop (seann/containers/Sequential.cu:121-130)
            model->forward(X);
            model->backward(label);
            losses[s] = model->lossFW(model->netY, label, lossBuf) / (float)batch;
            if (s == 0)
                for (const Slot& sl : slots)
                    cudaMemcpy(grads.data() + sl.offset, sl.p->grad()->elements, sizeof(float) * sl.p->data()->dims.size,
                               cudaMemcpyDeviceToHost);
            model->learn();
        }
        for (const Slot& sl : slots)
            cudaMemcpy(params.data() + sl.offset, sl.p->data()->elements, sizeof(float) * sl.p->data()->dims.size,
                       cudaMemcpyDeviceToHost);
        FILE* f = std::fopen(argv[10], "wb");
        if (!f) { std::fprintf(stderr, "cannot write %s\n", argv[10]); return 2; }
        std::fwrite(losses.data(), 4, losses.size(), f);
        std::fwrite(params.data(), 4, params.size(), f);
        std::fwrite(grads.data(), 4, grads.size(), f);
        std::fclose(f);
        std::printf("relink train ok: %zu operands, %zu parameter floats, loss %f -> %f\n", ops.size(), total, losses[0],
                    losses[steps - 1]);
        return 0;
    } catch (const std::exception& e) {
        std::fprintf(stderr, "relink_driver: %s\n", e.what());
        return 1;
    }
}
