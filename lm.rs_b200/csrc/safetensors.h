// safetensors.h -- read-only view of a safetensors file: 8-byte little-endian header length, that many bytes of JSON
// (tensor name -> dtype, shape, data_offsets relative to the end of the header), then the tensor data.  The file is
// mapped, not read: a loader copies each tensor to the device straight from the mapping.
#pragma once
#include <fcntl.h>
#include <stdint.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <map>
#include <string>
#include <vector>

#include "json.h"

namespace lmrs {

struct StTensor {
    std::string dtype;             // "BF16", "F32", "I32", ...
    std::vector<int64_t> shape;
    const uint8_t* data = nullptr;
    size_t bytes = 0;
    size_t numel() const { size_t n = 1; for (int64_t d : shape) n *= (size_t)d; return n; }
};

class SafeTensors {
  public:
    ~SafeTensors() { if (map_ && map_ != MAP_FAILED) munmap(map_, len_); }
    bool open(const std::string& path, std::string& err) {
        const int fd = ::open(path.c_str(), O_RDONLY);
        struct stat st;
        if (fd < 0 || fstat(fd, &st) != 0) { if (fd >= 0) close(fd); err = "cannot open " + path; return false; }
        len_ = (size_t)st.st_size;
        map_ = mmap(nullptr, len_, PROT_READ, MAP_PRIVATE, fd, 0);
        close(fd);
        if (map_ == MAP_FAILED) { map_ = nullptr; err = "cannot map " + path; return false; }
        const uint8_t* b = static_cast<const uint8_t*>(map_);
        if (len_ < 8) { err = path + ": too short for a safetensors file"; return false; }
        uint64_t hl = 0;
        for (int i = 7; i >= 0; i--) hl = (hl << 8) | b[i];
        if (hl > len_ - 8) { err = path + ": header length exceeds the file"; return false; }
        Json hdr;
        JsonParser jp(reinterpret_cast<const char*>(b + 8), (size_t)hl);
        if (!jp.parse(hdr, err) || !hdr.is_obj()) { err = path + ": header: " + err; return false; }
        const uint8_t* base = b + 8 + hl;
        const size_t room = len_ - 8 - (size_t)hl;
        for (const auto& kv : hdr.obj) {
            if (kv.first == "__metadata__") continue;
            const Json& t = kv.second;
            StTensor st_t;
            st_t.dtype = t.at("dtype").str;
            for (const Json& d : t.at("shape").arr) st_t.shape.push_back((int64_t)d.num);
            const Json& off = t.at("data_offsets");
            if (off.arr.size() != 2) { err = path + ": tensor '" + kv.first + "' has no data_offsets"; return false; }
            const size_t lo = (size_t)off.arr[0].num, hi = (size_t)off.arr[1].num;
            if (lo > hi || hi > room) { err = path + ": tensor '" + kv.first + "' lies outside the file"; return false; }
            st_t.data = base + lo;
            st_t.bytes = hi - lo;
            const size_t esz = st_t.dtype == "BF16" || st_t.dtype == "F16" ? 2 : (st_t.dtype == "F32" || st_t.dtype == "I32" ? 4 : (st_t.dtype == "F64" || st_t.dtype == "I64" ? 8 : 1));
            if (st_t.numel() * esz != st_t.bytes) { err = path + ": tensor '" + kv.first + "': shape and byte count disagree"; return false; }
            tensors_[kv.first] = st_t;
        }
        return true;
    }
    const StTensor* find(const std::string& name) const {
        auto it = tensors_.find(name);
        return it == tensors_.end() ? nullptr : &it->second;
    }
    const std::map<std::string, StTensor>& all() const { return tensors_; }

  private:
    void* map_ = nullptr;
    size_t len_ = 0;
    std::map<std::string, StTensor> tensors_;
};

}  // namespace lmrs
