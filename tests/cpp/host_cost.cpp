// What one materialisation costs the host through the C ABI, without any language binding on
// top: the nine-op fused chain of the first benchmark configuration,
//   y = cos(sin(x * 2 + 1)) * 0.5 + exp(-(x * x)),
// built as a lazy graph, resolved to one kernel and released, in a loop.  Run on the compile-only
// device (argument --compile-only-device: everything but the launch itself happens) or on GPU 0.
// Prints microseconds per pass for "build + release" and "build + materialise + release"; the
// crate pays graph walk, shader text, bind groups and one submit per kernel for the same request
// (src/compute_graph/resolve.rs:16-248, src/kernel.rs:244-389).
#include <chrono>
#include <cstdio>
#include <cstring>
#include <vector>

#include "wgf.h"

#define CK(x)                                                           \
    do {                                                                \
        const int r_ = (x);                                             \
        if (r_) {                                                       \
            std::printf("status %d at %s: %s\n", r_, #x, wgf_last_error()); \
            return 1;                                                   \
        }                                                               \
    } while (0)

int main(int argc, char** argv) {
    const bool dry = argc > 1 && std::strcmp(argv[1], "--compile-only-device") == 0;
    wgf_device* d;
    CK(wgf_device_create(dry ? -1 : 0, &d));
    const int64_t shape[2] = {1024, 1024};
    std::vector<float> host(1024 * 1024, 0.5f);
    wgf_tensor* x;
    CK(wgf_tensor_from_host(d, WGF_F32, 2, shape, host.data(), &x));
    auto chain = [&](bool materialise) -> int {
        wgf_tensor *a, *b, *c, *e, *f, *g, *h, *i, *y;
        CK(wgf_tensor_scalar(x, WGF_OP_MUL_C, 2.0f, &a));
        CK(wgf_tensor_scalar(a, WGF_OP_ADD_C, 1.0f, &b));
        CK(wgf_tensor_unary(b, WGF_OP_SIN, &c));
        CK(wgf_tensor_unary(c, WGF_OP_COS, &e));
        CK(wgf_tensor_scalar(e, WGF_OP_MUL_C, 0.5f, &f));
        CK(wgf_tensor_binary(x, x, WGF_OP_MUL, &g));
        CK(wgf_tensor_unary(g, WGF_OP_NEG, &h));
        CK(wgf_tensor_unary(h, WGF_OP_EXP, &i));
        CK(wgf_tensor_binary(f, i, WGF_OP_ADD, &y));
        if (materialise) CK(wgf_tensor_materialize(y));
        for (wgf_tensor* t : {a, b, c, e, f, g, h, i, y}) CK(wgf_tensor_release(t));
        return 0;
    };
    for (int k = 0; k < 200; ++k)
        if (chain(true)) return 1;
    if (!dry) CK(wgf_device_sync(d));
    const int n = 20000;
    const auto t0 = std::chrono::steady_clock::now();
    for (int k = 0; k < n; ++k)
        if (chain(false)) return 1;
    const auto t1 = std::chrono::steady_clock::now();
    for (int k = 0; k < n; ++k)
        if (chain(true)) return 1;
    if (!dry) CK(wgf_device_sync(d));
    const auto t2 = std::chrono::steady_clock::now();
    std::printf("host cost per pass: build + release %.2f us, build + materialise + release %.2f us (%s)\n",
                std::chrono::duration<double, std::micro>(t1 - t0).count() / n,
                std::chrono::duration<double, std::micro>(t2 - t1).count() / n, dry ? "compile-only device" : "GPU 0");
    CK(wgf_tensor_release(x));
    CK(wgf_device_release(d));
    std::printf("host cost ok\n");
    return 0;
}
