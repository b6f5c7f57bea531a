// Reader and writer of the reference's .crseq model files (seio/modelcache/codec.cu:8-97 with the per-operand records
// of seann/operands/**/encodeInfo / encodeNetParams and seann/containers/NetParam.cuh:41-112), so that weights trained
// by the reference load into this library's training executor and the other way round.
//
// Layout, all little-endian 32-bit words, written back to back (the reference opens the file in append mode, so its
// seekp offsets do not apply):
//   header        magic 0x7921aedf, operand count, epoch id
//   operand ids   one word per top-level operand
//   info records  in operand order. cuConv2D (0xd002) / Conv2D (0x0002): filter n, c, h, w, strideH, strideW, padH,
//                 padW, hasBias; Linear (0x0001): output size; AvgPool2D (0xb001): strideH, strideW, rangeH,
//                 rangeW; ShortcutEndpoint begin (0xf002): uuid, 0; end (0xf003): uuid, branch operand count, the
//                 branch operands' ids, then their info records; BatchNorm (0x0003), ReLU (0xa002), Softmax (0x0005),
//                 GlobalAvgPool (0xb002): nothing
//   parameters    in operand order, raw fp32: convolution filter [, bias]; BatchNorm beta, then gamma; Linear weights,
//                 then biases; ShortcutEndpoint end: its branch operands' parameters
// Host code only: nothing here touches the GPU except the copies between the file image and the bound parameter buffer.
#include <cstdio>
#include <cstring>
#include <fstream>
#include <string>
#include <vector>

#include "cb_internal.h"

namespace cb {

enum : uint32_t {
    CRSEQ_MAGIC = 0x7921aedfu,
    OPR_LINEAR = 0x0001, OPR_CONV2D = 0x0002, OPR_BATCHNORM = 0x0003, OPR_SOFTMAX = 0x0005, OPR_RELU = 0xa002,
    OPR_AVGPOOL2D = 0xb001, OPR_GLOBALAVGPOOL = 0xb002, OPR_CUCONV2D = 0xd002, OPR_SHORTCUT_BEG = 0xf002,
    OPR_SHORTCUT_END = 0xf003
};

bool crseq_parse(const std::vector<uint8_t>& file, CrseqModel& out, std::string& err) {
    size_t pos = 0;
    auto word = [&](uint32_t& v) -> bool {
        if (pos + 4 > file.size()) { err = "file ends inside a record"; return false; }
        std::memcpy(&v, file.data() + pos, 4);
        pos += 4;
        return true;
    };
    uint32_t magic = 0, count = 0;
    if (!word(magic) || !word(count) || !word(out.epoch)) return false;
    if (magic != CRSEQ_MAGIC) { err = "not a .crseq file (magic number)"; return false; }
    if (count > 1u << 20) { err = "implausible operand count"; return false; }
    std::vector<uint32_t> ids(count);
    for (uint32_t& id : ids)
        if (!word(id)) return false;
    // info records; `flat` lists every operand that owns records or parameters, branch operands after their endpoint
    std::vector<CrseqOperand> flat;
    auto read_info = [&](uint32_t id, CrseqOperand& o) -> bool {
        o = CrseqOperand{};
        o.id = id;
        switch (id) {
            case OPR_CUCONV2D: case OPR_CONV2D:
                for (int k = 0; k < 9; ++k)
                    if (!word(o.info[k])) return false;
                o.param_floats[0] = (uint64_t)o.info[0] * o.info[1] * o.info[2] * o.info[3];
                o.param_floats[1] = o.info[8] ? o.info[0] : 0;
                return true;
            case OPR_LINEAR: return word(o.info[0]);  // parameter sizes need the input width: resolved by the caller
            case OPR_AVGPOOL2D:
                for (int k = 0; k < 4; ++k)
                    if (!word(o.info[k])) return false;
                return true;
            case OPR_SHORTCUT_BEG: case OPR_SHORTCUT_END: return word(o.info[0]) && word(o.info[1]);
            case OPR_BATCHNORM: case OPR_RELU: case OPR_SOFTMAX: case OPR_GLOBALAVGPOOL: return true;
            default:
                err = "operand id 0x" + std::to_string(id) + " is outside the models this library trains";
                return false;
        }
    };
    for (uint32_t id : ids) {
        CrseqOperand o;
        if (!read_info(id, o)) return false;
        flat.push_back(o);
        if (id == OPR_SHORTCUT_END && o.info[1] > 0) {
            std::vector<uint32_t> branch(o.info[1]);
            for (uint32_t& b : branch)
                if (!word(b)) return false;
            for (uint32_t b : branch) {
                CrseqOperand bo;
                if (!read_info(b, bo)) return false;
                bo.in_branch = 1;
                flat.push_back(bo);
            }
        }
    }
    out.operands = flat;
    out.params_begin = pos;
    out.param_bytes = file.size() - pos;
    return true;
}

}  // namespace cb

using namespace cb;

extern "C" {

int cb_crseq_inspect(const char* path, unsigned* operand_count, unsigned* epoch, unsigned long long* param_floats, char* err,
                     int err_len) {
    auto failmsg = [&](const std::string& m) {
        if (err && err_len > 0) snprintf(err, (size_t)err_len, "%s", m.c_str());
        return CB_EINVAL;
    };
    if (!path) return failmsg("null path");
    std::ifstream f(path, std::ios::binary);
    if (!f) return failmsg(std::string("cannot open ") + path);
    std::vector<uint8_t> bytes((std::istreambuf_iterator<char>(f)), std::istreambuf_iterator<char>());
    CrseqModel mdl;
    std::string e;
    if (!crseq_parse(bytes, mdl, e)) return failmsg(e);
    if (operand_count) *operand_count = (unsigned)mdl.operands.size();
    if (epoch) *epoch = mdl.epoch;
    if (param_floats) *param_floats = mdl.param_bytes / 4;
    return CB_OK;
}

int cb_crseq_read_params(const char* path, float* out, unsigned long long count, char* err, int err_len) {
    auto failmsg = [&](const std::string& m) {
        if (err && err_len > 0) snprintf(err, (size_t)err_len, "%s", m.c_str());
        return CB_EINVAL;
    };
    if (!path || !out) return failmsg("null argument");
    std::ifstream f(path, std::ios::binary);
    if (!f) return failmsg(std::string("cannot open ") + path);
    std::vector<uint8_t> bytes((std::istreambuf_iterator<char>(f)), std::istreambuf_iterator<char>());
    CrseqModel mdl;
    std::string e;
    if (!crseq_parse(bytes, mdl, e)) return failmsg(e);
    if (count * 4 != mdl.param_bytes) return failmsg("the file holds " + std::to_string(mdl.param_bytes / 4) + " parameter floats");
    std::memcpy(out, bytes.data() + mdl.params_begin, mdl.param_bytes);
    return CB_OK;
}

}  // extern "C"
