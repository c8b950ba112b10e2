// Shared host-side types: status/error, element types, strided layouts.
#pragma once
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <memory>
#include <stdexcept>
#include <string>
#include <vector>

#include "../../include/wgf.h"

namespace wgf {

struct Error : std::exception {
    int code;
    std::string msg;
    Error(int c, std::string m) : code(c), msg(std::move(m)) {}
    const char* what() const noexcept override { return msg.c_str(); }
};

[[noreturn]] inline void fail(int code, const std::string& msg) { throw Error(code, msg); }

// Sets the calling thread's message returned by wgf_last_error() (defined in capi.cpp).
void set_last_error(const std::string& msg);

#define WGF_CHECK(cond, code, msg)                                   \
    do {                                                             \
        if (!(cond)) ::wgf::fail((code), std::string(msg));          \
    } while (0)

enum class DType : uint32_t { F32 = WGF_F32, F16 = WGF_F16, BF16 = WGF_BF16 };

inline size_t dtype_size(DType d) { return d == DType::F32 ? 4 : 2; }
inline const char* dtype_name(DType d) {
    switch (d) {
        case DType::F32: return "f32";
        case DType::F16: return "f16";
        default: return "bf16";
    }
}
inline bool valid_dtype(uint32_t d) { return d <= WGF_BF16; }

// Layout {offset, shape, strides} in elements; mirrors src/layout.rs:33-94 of the crate.
struct Layout {
    int64_t offset = 0;
    std::vector<int64_t> shape;
    std::vector<int64_t> strides;

    static std::vector<int64_t> contiguous_strides(const std::vector<int64_t>& shape) {
        std::vector<int64_t> s(shape.size());
        int64_t acc = 1;
        for (int i = (int)shape.size() - 1; i >= 0; --i) {
            s[i] = acc;
            acc *= shape[i];
        }
        return s;
    }
    static Layout contiguous(const std::vector<int64_t>& shape) {
        Layout l;
        l.shape = shape;
        l.strides = contiguous_strides(shape);
        return l;
    }
    int rank() const { return (int)shape.size(); }
    int64_t numel() const {
        int64_t n = 1;
        for (auto s : shape) n *= s;
        return n;
    }
    // Row-major strides (any offset).  Axes of extent 1 may carry any stride.
    bool is_dense() const {
        int64_t acc = 1;
        for (int i = rank() - 1; i >= 0; --i) {
            if (shape[i] != 1 && strides[i] != acc) return false;
            acc *= shape[i];
        }
        return true;
    }
    // The crate's definition: offset 0 and row-major strides (src/layout.rs:58-60).
    bool is_contiguous() const { return offset == 0 && is_dense(); }
    // True if two different indices can address the same element (src/layout.rs:86-90).
    bool allocation_overlaps() const {
        if (numel() == 0) return false;
        for (int i = 0; i < rank(); ++i)
            if (strides[i] == 0 && shape[i] > 1) return true;
        return false;
    }
    // Largest element index touched + 1 (relative to the buffer start).
    int64_t extent() const {
        if (numel() == 0) return offset;
        int64_t hi = offset;
        for (int i = 0; i < rank(); ++i) hi += (shape[i] - 1) * strides[i];
        return hi + 1;
    }
};

}  // namespace wgf
