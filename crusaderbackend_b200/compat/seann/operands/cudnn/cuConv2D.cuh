// The operand named cuConv2D, on this library's convolution kernels instead of cuDNN.
//
// The reference's model definitions (archive/Resnet56, seann/operands/prefabs/DenseBlock.cuh:51,58) build their
// convolutions from seann::cuConv2D (seann/operands/cudnn/cuConv2D.cuh:10-52). This header takes that file's place on
// the include path: same class name, constructor arguments, public members, operand id and .crseq record layout, with
// forward / xGrads / paramGrads lowered onto seblas::conv / convDerive / convError / channelReduce of the shim, i.e. the
// sm_100a tensor-core kernels. A second constructor accepts (and ignores) a leading cudnnHandle_t, which the archive
// model files still pass.
#pragma once
#include "../OperandBase.cuh"

#define OPR_CUDNN_CONV2D 0xd002

namespace seann {

class cuConv2D : public OperandBase {
public:
    shape4 filterShape;
    NetParam* filter{};
    NetParam* bias = nullptr;
    uint32 strideH, strideW, padH, padW;
    uint32 dilationH = 1, dilationW = 1;
    bool WITH_BIAS = true;

    cuConv2D(shape4 filterShape, uint32 strideH, uint32 strideW, uint32 padH, uint32 padW, bool WITH_BIAS)
        : filterShape(filterShape), strideH(strideH), strideW(strideW), padH(padH), padW(padW) {
        this->WITH_BIAS = WITH_BIAS;
    }
    cuConv2D(cudnnHandle_t, shape4 filterShape, uint32 strideH, uint32 strideW, uint32 padH, uint32 padW, bool WITH_BIAS)
        : cuConv2D(filterShape, strideH, strideW, padH, padW, WITH_BIAS) {}

    string info() override {
        return "cuConv2D        { filter: " + filterShape.toString() + ", input feature: " + X->A->dims.toString() + " }";
    }

    void initNetParams(OptimizerInfo* info, shape4 inShape) override {
        filter = (new NetParam(info, filterShape))->setWeight();
        if (WITH_BIAS) bias = new NetParam(info, filterShape.n, 1);
        X = Parameter::declare(inShape);
        assert(inShape.c == filterShape.c);
        Y = Parameter::create(shape4(inShape.n, filterShape.n, (inShape.h + 2 * padH - filterShape.h) / strideH + 1,
                                     (inShape.w + 2 * padW - filterShape.w) / strideW + 1));
    }
    void forward() override {
        conv(filter->data(), X->A, Y->A, (int)strideH, (int)strideW, (int)padH, (int)padW, WITH_BIAS ? bias->data() : nullptr);
    }
    void xGrads() override {
        *Y->dA + Y->dAReserve;
        convDerive(filter->data(), Y->dA, X->dA, (int)strideH, (int)strideW, (int)padH, (int)padW);
        Y->dAReserve->constFill(0);
    }
    // cuDNN's backward-filter call was made with beta = 0 (seann/operands/cudnn/cuConv2D.cu:67-79): the gradient is
    // assigned, not accumulated, so the filter gradient is cleared before the accumulating convError.
    void paramGrads() override {
        filter->grad()->constFill(0);
        convError(Y->dA, X->A, filter->grad(), (int)strideH, (int)strideW, (int)padH, (int)padW);
        if (WITH_BIAS) channelReduceBatch();
    }
    void updateParams() override { filter->opt->apply(); if (WITH_BIAS) bias->opt->apply(); }
    void batchUpdateParams() override { filter->opt->batchApply(); if (WITH_BIAS) bias->opt->batchApply(); }
    void randFillNetParams() override {
        const uint32 K = filter->data()->dims.size / filter->data()->dims.n;
        filter->data()->randNormal(0, (float)sqrt(2.0 / (float)K));
        if (WITH_BIAS) bias->data()->randNormal(0, (float)sqrt(2.0 / (float)filter->data()->dims.n));
    }
    void zeroGrads() override { filter->opt->zeroGrad(); if (WITH_BIAS) bias->opt->zeroGrad(); }

    uint32 OPERAND_ID() override { return OPR_CUDNN_CONV2D; }
    float getOptimLR() override { return filter->opt->LEARNING_RATE; }
    void updateOptimLR(float val) override { filter->opt->LEARNING_RATE = val; if (WITH_BIAS) bias->opt->LEARNING_RATE = val; }
    float getL2Const() override { return filter->opt->L2; }
    void updateL2Const(float val) override { filter->opt->L2 = val; if (WITH_BIAS) bias->opt->L2 = val; }

    // .crseq records: filter dims (4 x uint32) + strides, paddings, bias flag (5 x uint32); then the filter and bias
    // values. The file is opened in append mode by seio::saveSequence, so the records land back to back.
    uint32 encodeInfo(fstream* fout, uint64 offset) override {
        const uint32 n = WITH_BIAS ? 1 : 0;
        filter->encodeNetParamInfo(fout, offset);
        fout->write((char*)&strideH, sizeof(uint32));
        fout->write((char*)&strideW, sizeof(uint32));
        fout->write((char*)&padH, sizeof(uint32));
        fout->write((char*)&padW, sizeof(uint32));
        fout->write((char*)&n, sizeof(uint32));
        return sizeof(uint32) * 9;
    }
    uint32 encodeNetParams(fstream* fout, uint64 offset) override {
        uint32 written = filter->encodeNetParamData(fout, offset);
        if (WITH_BIAS) written += bias->encodeNetParamData(fout, offset + written);
        return written;
    }
    uint32 getInfoEncodingSize() override { return sizeof(uint32) * 9; }
    uint32 getNetParamsEncodingSize() override {
        return (filter->data()->dims.size + (WITH_BIAS ? bias->data()->dims.size : 0)) * sizeof(float);
    }

private:
    // bias gradient = sum of dY over (n, h, w) per channel (cudnnConvolutionBackwardBias with beta = 0)
    void channelReduceBatch() {
        SEBLAS_CB(cb_conv_bias_grad(seblas::context(), Y->dA->elements, bias->grad()->elements, (int)Y->dA->dims.n,
                                    (int)Y->dA->dims.c, (int)(Y->dA->dims.h * Y->dA->dims.w), 0));
    }
};

}  // namespace seann
