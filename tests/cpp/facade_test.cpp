// The crate's own tests, restated against the C++ mirror of its API (include/wgf/tensor.hpp).
// Each block cites the test it follows.  Exit code 0 and "facade ok" on success.
#include <cmath>
#include <cstdio>
#include <cstdlib>

#include "wgf/tensor.hpp"

using wgf::Device;
using wgf::Tensor;

#define EXPECT(cond)                                                        \
    do {                                                                    \
        if (!(cond)) {                                                      \
            std::fprintf(stderr, "%s:%d: failed: %s\n", __FILE__, __LINE__, #cond); \
            std::exit(1);                                                   \
        }                                                                   \
    } while (0)

int main(int argc, char** argv) {
    const bool compile_only = argc > 1 && std::string(argv[1]) == "--compile-only-device";
    Device device(compile_only ? -1 : 0);
    auto data = Tensor<2, float>::from_rows(device, {{1.f, 2.f}, {3.f, 4.f}, {5.f, 6.f}});

    // src/element_wise.rs:214-262 test_add_const
    auto plus = data + 1.0f;
    // src/reduce.rs:570-599 test_reduce_const_add_then_sum_fused
    auto fused = (data + 1.0f).sum(0);
    // src/reduce.rs:604-631 test_reduce_const_sum_then_add_fused
    auto after = data.sum(1) + 1.0f;
    // src/composite/rms_norm.rs:20-40 test_layer_norm
    auto weight = Tensor<1, float>::from_values(device, {2.f, 3.f});
    auto normed = data.layer_norm(weight, 1e-5f);
    // src/composite/cat.rs:45-78 test_cat
    auto other = Tensor<2, float>::from_rows(device, {{1.f, -2.f}, {-3.f, 4.f}, {5.f, -6.f}});
    auto joined = Tensor<2, float>::cat({other, data}, 1);
    // src/matmul.rs:219-239 test_matmul
    auto a = Tensor<2, float>::from_rows(device, {{1.f}, {3.f}});
    auto b = Tensor<2, float>::from_rows(device, {{1.f, 2.f}});
    auto prod = a.mat_mul(b);
    // src/map_layout.rs:103-149 test_transpose / test_broadcast
    auto tr = data.transpose(0, 1);
    auto bc = Tensor<2, float>::from_rows(device, {{1.f, 2.f}, {3.f, 4.f}}).broadcast({2, 2, 3});
    // src/element_wise.rs:1440-1499 casts
    auto half = data.cast<wgf::f16>().cast<float>();
    // examples/hello.rs:15-22
    std::vector<float> ones(10 * 10 * 20, 1.f);
    Tensor<3, float> big(device, {10, 10, 20}, ones.data());
    auto total = big.sum(0).sum(0).sum(0);
    // beyond the crate: two results as one request (the reduction rides along in the row kernel)
    auto probs = data.softmax_last_dim();
    auto sum_all = data.sum(0).sum(0);
    wgf::materialize_all(probs, sum_all);

    EXPECT((joined.shape() == std::array<int64_t, 2>{3, 4}));
    EXPECT((bc.shape() == std::array<int64_t, 3>{2, 2, 3}));
    EXPECT((total.shape() == std::array<int64_t, 0>{}));
    bool threw = false;
    try {
        auto bad = data + tr;   // [3,2] + [2,3]: the crate asserts equal shapes, src/pair_wise.rs:92
    } catch (const wgf::Error& e) {
        threw = e.code == WGF_ERR_SHAPE;
    }
    EXPECT(threw);

    // beyond the crate: a materialisation recorded once and replayed
    auto feed = wgf::Tensor<2, float>::from_rows(device, {{1.f, 2.f}, {3.f, 4.f}, {5.f, 6.f}});
    const uint64_t before_recording = device.launch_count();
    wgf::Schedule schedule(device);
    auto doubled = feed * 2.f;
    auto row_sums = doubled.sum(1);
    doubled.materialize();
    row_sums.materialize();
    bool refused = false;
    try {
        doubled.as_slice();   // nothing has run yet: a recording refuses downloads
    } catch (const wgf::Error& e) {
        refused = e.code == WGF_ERR_UNSUPPORTED;
    }
    EXPECT(refused);
    schedule.finish();
    EXPECT(schedule.kernel_count() == 2 && device.launch_count() - before_recording == 2);
    const float next[6] = {10.f, 20.f, 30.f, 40.f, 50.f, 60.f};
    feed.write(next);
    schedule.launch();
    EXPECT(device.launch_count() - before_recording == 4);

    if (compile_only) {
        std::printf("facade ok (compile-only device)\n");
        return 0;
    }

    auto p = plus.as_slice();
    EXPECT((p[{0, 0}] == 2.f && p[{0, 1}] == 3.f && p[{2, 1}] == 7.f));
    auto f = fused.as_slice();
    EXPECT((f[{0}] == 12.f && f[{1}] == 15.f));
    auto s = after.as_slice();
    EXPECT((s[{0}] == 4.f && s[{1}] == 8.f && s[{2}] == 12.f));
    auto n = normed.as_slice();
    const float want[3][2] = {{1.2649086f, 3.7947257f}, {1.6970556f, 3.3941112f}, {1.8107147f, 3.2592864f}};
    for (int i = 0; i < 3; ++i)
        for (int j = 0; j < 2; ++j) EXPECT(std::fabs(n[{i, j}] - want[i][j]) < 1e-3f);
    auto j = joined.as_slice();
    EXPECT((j[{0, 0}] == 1.f && j[{0, 1}] == -2.f && j[{0, 2}] == 1.f && j[{2, 3}] == 6.f));
    auto m = prod.as_slice();
    EXPECT((m[{0, 0}] == 1.f && m[{0, 1}] == 2.f && m[{1, 0}] == 3.f && m[{1, 1}] == 6.f));
    auto t = tr.as_slice();
    EXPECT((t[{0, 2}] == 5.f && t[{1, 0}] == 2.f));
    auto c = bc.as_slice();
    EXPECT((c[{0, 1, 2}] == 2.f && c[{1, 0, 0}] == 3.f));
    EXPECT((half.as_slice() == data.as_slice()));
    EXPECT((total.as_slice()[{}] == 2000.f));
    EXPECT(!total.all_timing_information().empty());
    EXPECT((sum_all.as_slice()[{}] == 21.f));
    auto replayed = row_sums.as_slice();   // the values of the replay, from the data written before it
    EXPECT((replayed[{0}] == 60.f && replayed[{1}] == 140.f && replayed[{2}] == 220.f));
    EXPECT((doubled.as_slice()[{2, 1}] == 120.f));
    auto pr = probs.as_slice();
    EXPECT(std::fabs(pr[{1, 0}] + pr[{1, 1}] - 1.f) < 1e-6f);

    // tests/inplace_clone.rs:6-37: an in-place optimisation must not change a tensor that is still held
    for (int round = 0; round < 2; ++round) {
        auto again = Tensor<2, float>(data) + 1.0f;   // clone, then consume the clone
        EXPECT((again.as_slice()[{1, 1}] == 5.f));
    }
    EXPECT((data.as_slice()[{1, 1}] == 4.f));
    std::printf("facade ok\n");
    return 0;
}
