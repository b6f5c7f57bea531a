// In-memory synthetic stand-in for the reference's seio/data/Dataset.cuh (which reads image files through OpenCV and
// Windows paths): the members and calls that seann::Sequential::train touches (seann/containers/Sequential.cu:107-161)
// over seeded N(0,1) images and uniform one-hot labels — BATCH_SIZE, MINI_BATCH_SIZE, MAX_EPOCH, TEST_SIZE, batchID,
// epochID, dataBatch[2][..]->{X,label}, testset[..]->{X,label}, genBatch(), genBatchAsync(), procDisplay.
#pragma once
#include <random>
#include <thread>
#include <vector>

#include "../../seblas/seblas.cuh"

using namespace seblas;
namespace seio {

struct Data {
    Tensor* X;
    Tensor* label;
    static Data* declare(shape4 dataShape, shape4 labelShape) {
        Data* d = new Data();
        d->X = Tensor::declare(dataShape);
        d->label = Tensor::declare(labelShape);
        return d;
    }
    Data* instantiate() { X->instantiate(); label->instantiate(); return this; }
};

// Console progress display of the reference (seio/watchDog/TrainProcDisplay.cuh), reduced to counters and one line per
// update.
class ProcDisplay {
public:
    const char* LOSS_TYPE;
    float epochTrainLoss = 0;
    float epochValidLoss = 0;
    float batchID = 0;
    explicit ProcDisplay(const char* lossType) : LOSS_TYPE(lossType) {}
    void show(uint32 epochID) { if (!logQuiet()) std::printf("epoch %u (%s)\n", epochID, LOSS_TYPE); }
    void update(float trainLoss, float validLoss) {
        epochTrainLoss += trainLoss;
        epochValidLoss += validLoss;
        batchID += 1;
        if (!logQuiet()) std::printf("  batch %.0f train loss %f valid loss %f\n", batchID, trainLoss, validLoss);
    }
    void reset() { epochTrainLoss = epochValidLoss = batchID = 0; }
};

struct Dataset {
public:
    Data** dataBatch[2];
    Data** testset = nullptr;
    uint32 BATCH_SIZE, EPOCH_SIZE, MAX_EPOCH, MINI_BATCH_SIZE, TEST_SIZE = 0;
    uint32 batchID = 0;
    uint32 epochID = 0;
    shape4 dataShape;
    shape4 labelShape;
    ProcDisplay* procDisplay;
    std::mt19937_64 rng;

    // Same argument order as the reference's Dataset::construct (seio/data/Dataset.cuh:53-54); dataShape is one sample
    // (c, h, w), labelShape (classes, 1).
    static Dataset* construct(uint32 batchSize, uint32 miniBatchSize, uint32 epochSize, uint32 maxEpoch, shape4 dataShape,
                              shape4 labelShape) {
        Dataset* d = new Dataset(dataShape, labelShape);
        d->BATCH_SIZE = batchSize; d->MINI_BATCH_SIZE = miniBatchSize; d->EPOCH_SIZE = epochSize; d->MAX_EPOCH = maxEpoch;
        d->procDisplay = new ProcDisplay("cross entropy");
        const uint32 minis = batchSize / miniBatchSize;
        for (int b = 0; b < 2; ++b) {
            d->dataBatch[b] = new Data*[minis];
            for (uint32 i = 0; i < minis; ++i)
                d->dataBatch[b][i] = Data::declare(shape4(miniBatchSize, dataShape.c, dataShape.h, dataShape.w),
                                                   shape4(miniBatchSize, 1, labelShape.h, labelShape.w))->instantiate();
        }
        return d;
    }
    void setSeed(uint64 seed) { rng.seed(seed); }
    void setProcDispaly(ProcDisplay* display) { procDisplay = display; }
    void allocTestSet(uint32 testSize) {
        TEST_SIZE = testSize;
        const uint32 minis = testSize / MINI_BATCH_SIZE;
        testset = new Data*[minis];
        for (uint32 i = 0; i < minis; ++i) {
            testset[i] = Data::declare(shape4(MINI_BATCH_SIZE, dataShape.c, dataShape.h, dataShape.w),
                                       shape4(MINI_BATCH_SIZE, 1, labelShape.h, labelShape.w))->instantiate();
            fill(testset[i]);
        }
    }
    // Fills the buffer the NEXT training pass will read and advances the counters the way the reference's loader does.
    void genBatch() {
        const uint32 minis = BATCH_SIZE / MINI_BATCH_SIZE;
        for (uint32 i = 0; i < minis; ++i) fill(dataBatch[batchID % 2][i]);
        batchID++;
        if ((uint64)batchID * BATCH_SIZE >= (uint64)(epochID + 1) * EPOCH_SIZE) epochID++;
    }
    std::thread genBatchAsync() { return std::thread([this] { genBatch(); }); }

private:
    Dataset(shape4 d, shape4 l) : dataShape(d), labelShape(l), rng(0x5eedull) {}
    void fill(Data* d) {
        std::normal_distribution<float> nd(0.f, 1.f);
        std::vector<float> x(d->X->dims.size), lab(d->label->dims.size, 0.f);
        for (float& v : x) v = nd(rng);
        const uint32 classes = d->label->dims.size / d->label->dims.n;
        for (uint32 n = 0; n < d->label->dims.n; ++n) lab[(size_t)n * classes + rng() % classes] = 1.f;
        cudaMemcpy(d->X->elements, x.data(), x.size() * sizeof(float), cudaMemcpyHostToDevice);
        cudaMemcpy(d->label->elements, lab.data(), lab.size() * sizeof(float), cudaMemcpyHostToDevice);
    }
};

}  // namespace seio
