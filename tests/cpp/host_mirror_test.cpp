// Exercises the C++ host mirror (include/kore_b200.hpp) the way the reference's own unit tests
// exercise BitLinear / QuatLinear / the kernel functions, and checks the CUDA results against
// the CPU restatement (libkbref, test infrastructure) bit for bit.  Built and run by
// tests/test_cpp_host_mirror.py; prints "OK <checks>" on success.
#include <cmath>
#include <cstdio>
#include <cstring>
#include <random>

#include "kore_b200.hpp"
#include "kbref.h"

using namespace kore_b200;

static int checks = 0;
#define EXPECT(cond)                                                                  \
    do {                                                                              \
        ++checks;                                                                     \
        if (!(cond)) { std::printf("FAILED %s:%d: %s\n", __FILE__, __LINE__, #cond); return 1; } \
    } while (0)

static std::vector<float> gaussian(unsigned seed, size_t n, float sigma) {
    std::mt19937 g(seed);
    std::normal_distribution<float> d(0.0f, sigma);
    std::vector<float> v(n);
    for (auto &x : v) x = d(g);
    return v;
}

int main() {
    // bit_linear.rs:334-353: weights [[1,-1,0,1],[-1,1,1,0]], x = [1,2,3,4] -> 3, 4
    {
        const float w[8] = {1, -1, 0, 1, -1, 1, 1, 0};
        BitLinear l = BitLinear::create(w, nullptr, 2, 4, 0.3f);
        EXPECT(l.in_features() == 4 && l.out_features() == 2 && !l.has_bias());
        std::vector<size_t> oshape;
        auto y = l.forward({1, 2, 3, 4}, {4}, &oshape);
        EXPECT(oshape.size() == 1 && oshape[0] == 2);
        EXPECT(std::fabs(y[0] - 3.0f) < 0.5f && std::fabs(y[1] - 4.0f) < 0.5f);
        EXPECT(l.to_string().find("BitLinear(in=4, out=2, bias=false") == 0);
        // shape behaviour (:304-316): 2-D and 3-D inputs keep their leading dimensions
        auto y2 = l.forward(std::vector<float>(3 * 4, 1.0f), {3, 4}, &oshape);
        EXPECT(oshape == (std::vector<size_t>{3, 2}) && y2.size() == 6);
        auto y3 = l.forward(std::vector<float>(2 * 3 * 4, 1.0f), {2, 3, 4}, &oshape);
        EXPECT(oshape == (std::vector<size_t>{2, 3, 2}) && y3.size() == 12);
        // wrong last dimension -> ShapeMismatch (:179-184)
        bool threw = false;
        try { l.forward(std::vector<float>(5, 1.0f), {5}); } catch (const KoreError &e) { threw = e.kind() == KoreError::ShapeMismatch; }
        EXPECT(threw);
    }
    // seeded layer vs the restated W2A8 arithmetic, both kinds, several token counts (GEMV, small-batch, GEMM)
    const size_t m = 200, k = 333;
    auto w = gaussian(11, m * k, 0.02f);
    auto bias = gaussian(12, m, 0.1f);
    for (int kind = 0; kind < 2; ++kind) {
        std::vector<uint8_t> packed(m * (kind == 0 ? (k + 4) / 5 : (k + 3) / 4));
        std::vector<float> scales(m);
        if (kind == 0) kbref_pack_weights_ternary(w.data(), m, k, 0.3f, packed.data(), scales.data());
        else kbref_pack_weights_quaternary(w.data(), m, k, packed.data(), scales.data());
        for (size_t n : {size_t(1), size_t(7), size_t(150)}) {
            auto x = gaussian(20 + (unsigned)n, n * k, 1.0f);
            std::vector<float> y_ref(n * m);
            std::vector<int32_t> acc_ref(n * m);
            EXPECT(kbref_q_forward(kind, packed.data(), scales.data(), bias.data(), m, k, x.data(), n, y_ref.data(), acc_ref.data(), 2) == 0);
            std::vector<float> y;
            if (kind == 0) {
                BitLinear l = BitLinear::from_packed(packed, scales, bias.data(), k, m);
                y = l.forward(x, {n, k});
                EXPECT(l.packed_weights() == packed && l.scales() == scales);
                EXPECT(l.compression_ratio() > 5.0f);
            } else {
                QuatLinear l = QuatLinear::from_packed(packed, scales, bias.data(), k, m);
                y = l.forward(x, {n, k});
                EXPECT(l.packed_weights() == packed);
                std::vector<float> wd(m * k);
                kbref_dequantize_quaternary(packed.data(), scales.data(), m, k, wd.data());
                EXPECT(l.dequantize_weights() == wd);
            }
            EXPECT(std::memcmp(y.data(), y_ref.data(), y.size() * sizeof(float)) == 0);
        }
    }
    // device-side quantiser of BitLinear::create == the restated packer
    {
        auto [p_gpu, s_gpu] = pack_weights_ternary(w, m, k, 0.3f);
        std::vector<uint8_t> p(m * ((k + 4) / 5));
        std::vector<float> s(m);
        kbref_pack_weights_ternary(w.data(), m, k, 0.3f, p.data(), s.data());
        EXPECT(p_gpu == p && s_gpu == s);
        auto [q_gpu, t_gpu] = pack_weights_quaternary(w, m, k);
        std::vector<uint8_t> q(m * ((k + 3) / 4));
        kbref_pack_weights_quaternary(w.data(), m, k, q.data(), s.data());
        EXPECT(q_gpu == q && t_gpu == s);
    }
    // kernel-shaped one-shots with integer activations and unit scales: identical to the f32 reference arithmetic
    {
        const size_t mm = 16, kk = 32, nn = 16;
        auto ww = gaussian(31, mm * kk, 0.02f);
        std::vector<uint8_t> p(mm * ((kk + 4) / 5));
        std::vector<float> s(mm), ones(mm, 1.0f);
        kbref_pack_weights_ternary(ww.data(), mm, kk, 0.3f, p.data(), s.data());
        std::vector<float> b(kk * nn);
        std::mt19937 g(5);
        for (auto &v : b) v = (float)((int)(g() % 255) - 127);
        std::vector<float> c_ref(mm * nn);
        EXPECT(kbref_ternary_matmul(p.data(), p.size(), ones.data(), mm, b.data(), c_ref.data(), mm, nn, kk, 1) == 0);
        // per-token absmax must be 127 for the quantiser to be the identity: force one 127 per column
        for (size_t j = 0; j < nn; ++j) b[j] = 127.0f;
        EXPECT(kbref_ternary_matmul(p.data(), p.size(), ones.data(), mm, b.data(), c_ref.data(), mm, nn, kk, 1) == 0);
        auto c = ternary_matmul(p, ones, b, mm, nn, kk);
        EXPECT(c == c_ref);
        bool threw = false;
        try { p.pop_back(); ternary_matmul(p, ones, b, mm, nn, kk); } catch (const KoreError &e) {
            threw = e.kind() == KoreError::StorageError && std::string(e.what()).find("a_packed too small") == 0;
        }
        EXPECT(threw);
    }
    // both operands ternary (cpu_ternary_matmul.rs:293-307)
    {
        std::vector<float> a = {1, -1, 0, 1}, b = {1, 0, -1, 1};
        auto [pa, sa] = pack_weights_ternary(a, 2, 2, 0.3f);
        auto [pb, sb] = pack_weights_ternary(b, 2, 2, 0.3f);
        auto c = ternary_ternary_matmul(pa, sa, pb, sb, 2, 2, 2);
        EXPECT(c == (std::vector<float>{1, -2, 0, 1}));
    }
    // a group of same-shaped layers; members of another shape are a ShapeMismatch
    {
        const float w[8] = {1, -1, 0, 1, -1, 1, 1, 0};
        BitLinear a = BitLinear::create(w, nullptr, 2, 4, 0.3f), b = BitLinear::create(w, nullptr, 2, 4, 0.3f);
        BitLinear c = BitLinear::create(w, nullptr, 4, 2, 0.3f);
        LinearGroup g({&a, &b});
        EXPECT(g.size() == 2);
        bool threw = false;
        try { LinearGroup bad({&a, &c}); } catch (const KoreError &e) { threw = e.kind() == KoreError::ShapeMismatch; }
        EXPECT(threw);
    }
    std::printf("OK %d\n", checks);
    return 0;
}
