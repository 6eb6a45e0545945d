// GGUF v3 subset reader for the B200 decode engine (host side, C++17, no deps).
//
// Accepts exactly the on-disk subset that the reference reader accepts
// (reference src/gguf.h:183-222): little-endian header {magic, version,
// n_tensors, n_kv}; key/value pairs of scalar, string and array type (only the
// string array "tokenizer.ggml.tokens" is counted, its length is the vocabulary
// size: reference src/cpu_infer.cpp:79); tensor infos {name, n_dims, dims, type,
// offset}; tensor data at the next multiple of general.alignment (default 32).
// The engine itself needs only F32 and Q4_0 tensors; any other tensor type is
// reported as an error string instead of terminating the process.
#pragma once
#include <cstdint>
#include <cstring>
#include <string>
#include <unordered_map>
#include <vector>
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

namespace mib200 {

enum : uint32_t { GGML_F32 = 0, GGML_F16 = 1, GGML_Q4_0 = 2, GGML_Q4_1 = 3, GGML_Q8_0 = 8, GGML_Q6_K = 14 };

struct GgufTensor {
    uint32_t type = 0;
    std::vector<int64_t> ne;          // ne[0] = contiguous (in) dim, ne[1] = rows (out)
    const uint8_t* data = nullptr;
    int64_t cols() const { return ne.empty() ? 0 : ne[0]; }
    int64_t rows() const { int64_t r = 1; for (size_t i = 1; i < ne.size(); i++) r *= ne[i]; return r; }
    // bytes, or 0 for a type this engine does not size
    size_t nbytes() const {
        switch (type) {
            case GGML_F32: return (size_t)rows() * cols() * 4;
            case GGML_F16: return (size_t)rows() * cols() * 2;
            case GGML_Q4_0: return (size_t)rows() * (cols() / 32) * 18;
            case GGML_Q4_1: return (size_t)rows() * (cols() / 32) * 20;
            case GGML_Q8_0: return (size_t)rows() * (cols() / 32) * 34;
            case GGML_Q6_K: return (size_t)rows() * (cols() / 256) * 210;
            default: return 0;
        }
    }
};

class GgufFile {
public:
    GgufFile() = default;
    GgufFile(const GgufFile&) = delete;
    GgufFile& operator=(const GgufFile&) = delete;
    ~GgufFile() { close_file(); }

    // Returns an empty string on success, else a description of what is wrong.
    std::string open(const std::string& path) {
        close_file();
        fd_ = ::open(path.c_str(), O_RDONLY);
        if (fd_ < 0) return "cannot open " + path;
        struct stat st; if (fstat(fd_, &st) != 0) return "cannot stat " + path;
        size_ = (size_t)st.st_size;
        if (size_ < 24) return "file too short for a GGUF header";
        void* p = mmap(nullptr, size_, PROT_READ, MAP_PRIVATE, fd_, 0);
        if (p == MAP_FAILED) { base_ = nullptr; return "mmap failed"; }
        base_ = (const uint8_t*)p; cur_ = base_; end_ = base_ + size_; bad_ = false;

        if (rd<uint32_t>() != 0x46554747u) return "not a GGUF file (bad magic)";
        (void)rd<uint32_t>();                                   // version: ignored, as in the reference
        const uint64_t n_tensors = rd<uint64_t>(), n_kv = rd<uint64_t>();
        if (n_tensors > (1u << 24) || n_kv > (1u << 24)) return "implausible header counts";
        for (uint64_t i = 0; i < n_kv && !bad_; i++) {
            std::string key = rd_str();
            uint32_t vt = rd<uint32_t>();
            std::string e = rd_value(vt, key, 0);
            if (!e.empty()) return e;
        }
        struct Info { std::string name; GgufTensor t; uint64_t off; };
        std::vector<Info> infos; infos.reserve(n_tensors);
        for (uint64_t i = 0; i < n_tensors && !bad_; i++) {
            Info in; in.name = rd_str();
            uint32_t nd = rd<uint32_t>();
            if (nd > 4) return "tensor " + in.name + ": more than 4 dims";
            in.t.ne.resize(nd);
            for (uint32_t d = 0; d < nd; d++) in.t.ne[d] = (int64_t)rd<uint64_t>();
            in.t.type = rd<uint32_t>(); in.off = rd<uint64_t>();
            infos.push_back(std::move(in));
        }
        if (bad_) return "truncated GGUF metadata";
        uint64_t align = (uint64_t)num("general.alignment", 32);
        if (align == 0) align = 32;
        size_t pos = (size_t)(cur_ - base_);
        size_t data_start = (pos + align - 1) / align * align;
        if (data_start > size_) return "tensor data would start past the end of the file";
        for (auto& in : infos) {
            // a crafted file must not get past these with wrapped arithmetic: every dimension positive and at most
            // 2^31, the element count at most 2^40 (so the byte count cannot overflow), offset and size each checked
            // against what is left of the file
            unsigned long long elems = 1;
            for (int64_t d : in.t.ne) {
                if (d <= 0 || d > (1ll << 31)) return "tensor " + in.name + ": dimension out of range";
                elems *= (unsigned long long)d;
                if (elems > (1ull << 40)) return "tensor " + in.name + ": implausibly large";
            }
            const size_t nb = in.t.nbytes(), room = size_ - data_start;
            if (in.off > room || nb > room - in.off) return "tensor " + in.name + " runs past the end of the file";
            in.t.data = base_ + data_start + in.off;
            tensors_.emplace(in.name, in.t);
        }
        return "";
    }

    double num(const std::string& k, double def) const { auto it = num_.find(k); return it == num_.end() ? def : it->second; }
    bool has_num(const std::string& k) const { return num_.count(k) > 0; }
    const std::string& str(const std::string& k) const { static std::string e; auto it = str_.find(k); return it == str_.end() ? e : it->second; }
    size_t n_tokens() const { return n_tokens_; }
    const std::vector<std::string>& tokens() const { return tokens_; }
    bool has(const std::string& n) const { return tensors_.count(n) > 0; }
    const GgufTensor* find(const std::string& n) const { auto it = tensors_.find(n); return it == tensors_.end() ? nullptr : &it->second; }
    const std::unordered_map<std::string, GgufTensor>& tensors() const { return tensors_; }
    void keep_token_strings(bool k) { keep_tokens_ = k; }

private:
    int fd_ = -1; size_t size_ = 0;
    const uint8_t *base_ = nullptr, *cur_ = nullptr, *end_ = nullptr;
    bool bad_ = false, keep_tokens_ = false;
    size_t n_tokens_ = 0;
    std::unordered_map<std::string, double> num_;
    std::unordered_map<std::string, std::string> str_;
    std::vector<std::string> tokens_;
    std::unordered_map<std::string, GgufTensor> tensors_;

    void close_file() {
        if (base_) munmap((void*)base_, size_);
        if (fd_ >= 0) ::close(fd_);
        base_ = nullptr; fd_ = -1; num_.clear(); str_.clear(); tokens_.clear(); tensors_.clear(); n_tokens_ = 0;
    }
    template <typename T> T rd() {
        T v{};
        if (bad_ || cur_ + sizeof(T) > end_) { bad_ = true; return v; }
        memcpy(&v, cur_, sizeof(T)); cur_ += sizeof(T); return v;
    }
    std::string rd_str() {
        uint64_t n = rd<uint64_t>();
        if (bad_ || n > (uint64_t)(end_ - cur_)) { bad_ = true; return ""; }
        std::string s((const char*)cur_, (size_t)n); cur_ += n; return s;
    }
    void skip_str() {
        uint64_t n = rd<uint64_t>();
        if (bad_ || n > (uint64_t)(end_ - cur_)) { bad_ = true; return; }
        cur_ += n;
    }
    std::string rd_value(uint32_t vt, const std::string& key, int depth) {
        switch (vt) {
            case 0: num_[key] = rd<uint8_t>(); break;
            case 1: num_[key] = rd<int8_t>(); break;
            case 2: num_[key] = rd<uint16_t>(); break;
            case 3: num_[key] = rd<int16_t>(); break;
            case 4: num_[key] = rd<uint32_t>(); break;
            case 5: num_[key] = rd<int32_t>(); break;
            case 6: num_[key] = rd<float>(); break;
            case 7: num_[key] = rd<uint8_t>(); break;
            case 8: if (key.empty()) skip_str(); else str_[key] = rd_str(); break;
            case 10: num_[key] = (double)rd<uint64_t>(); break;
            case 11: num_[key] = (double)rd<int64_t>(); break;
            case 12: num_[key] = rd<double>(); break;
            case 9: {
                if (depth > 2) return "nested arrays too deep";
                uint32_t et = rd<uint32_t>(); uint64_t n = rd<uint64_t>();
                bool tok = (key == "tokenizer.ggml.tokens" && et == 8);
                if (tok) n_tokens_ = (size_t)n;
                for (uint64_t i = 0; i < n && !bad_; i++) {
                    if (et == 8) { if (tok && keep_tokens_) tokens_.push_back(rd_str()); else skip_str(); }
                    else { std::string e = rd_value(et, "", depth + 1); if (!e.empty()) return e; }
                }
                break;
            }
            default: return "bad metadata type " + std::to_string(vt);
        }
        num_.erase("");
        return bad_ ? "truncated GGUF metadata" : "";
    }
};

}  // namespace mib200
