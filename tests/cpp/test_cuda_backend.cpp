// C++ host test of the drop-in boundary: drives agn::CudaBackend (include/agention_b200.hpp)
// the way the reference's model code drives WgpuBackend::launch_*, and checks every result
// against the CPU oracle (oracle/cpu_ref.h, the checker only).  Exit code 0 = all parity
// checks passed.  Built and run by tests/test_gpu_cpp_host.py.
#include <cmath>
#include <cstdio>
#include <cstring>
#include <random>
#include <vector>

#include "agention_b200.hpp"
#include "cpu_ref.h"

static int failures = 0;

static double rel_to_row_scale(const std::vector<float> &got, const std::vector<float> &ref, size_t row_len) {
    double worst = 0.0;
    for (size_t r = 0; r * row_len < ref.size(); r++) {
        double scale = 1e-30;
        for (size_t i = 0; i < row_len; i++) scale = std::fmax(scale, std::fabs((double)ref[r * row_len + i]));
        for (size_t i = 0; i < row_len; i++)
            worst = std::fmax(worst, std::fabs((double)got[r * row_len + i] - (double)ref[r * row_len + i]) / scale);
    }
    return worst;
}

static void expect(bool ok, const char *what, double v = 0.0) {
    std::printf("%-28s %s (%.3g)\n", what, ok ? "ok" : "FAIL", v);
    if (!ok) failures++;
}

int main() {
    const double TOL = 1e-5;
    const int64_t T = 48, H = 3584, hd = 128, nq = 28, nkv = 4, I = 4096, vocab = 512;
    std::mt19937 rng(20261125);
    std::normal_distribution<float> N01(0.f, 1.f);
    auto randn = [&](size_t n) { std::vector<float> v(n); for (auto &x : v) x = N01(rng); return v; };
    auto weight = [&](size_t n) { std::vector<float> v(n); for (auto &x : v) x = 1.f + 0.02f * N01(rng); return v; };

    agn::CudaBackend be(0);
    std::printf("backend: %s\n", be.name());

    {  // rms_norm
        auto x = randn(T * H), w = weight(H);
        std::vector<float> ref(T * H);
        orc_rms_norm_rows(x.data(), w.data(), ref.data(), T, H, 1e-6f, 1);
        auto dx = be.upload(x), dw = be.upload(w);
        auto out = be.launch_rms_norm(dx.as<float>(), dw.as<float>(), T, H, 1e-6f);
        double e = rel_to_row_scale(be.read<float>(out, T * H), ref, H);
        expect(e <= TOL, "launch_rms_norm", e);
    }
    {  // rope on Q and K, then fused norm->rope
        auto q = randn(T * nq * hd), k = randn(T * nkv * hd), wq = weight(hd);
        std::vector<int32_t> pos(T);
        for (int64_t t = 0; t < T; t++) pos[t] = (int32_t)((t * 7919) % 32768);
        auto rq = q, rk = k;
        orc_rope_rows(rq.data(), T, nq, hd, hd, pos.data(), 1e6f, 1.f, ORC_ROPE_NEOX, 1);
        orc_rope_rows(rk.data(), T, nkv, hd, hd, pos.data(), 1e6f, 1.f, ORC_ROPE_NEOX, 1);
        auto dq = be.upload(q), dk = be.upload(k);
        auto dp = be.upload(pos);
        be.launch_rope_qk(dq.as<float>(), dk.as<float>(), T, nq, nkv, hd, hd, dp.as<int32_t>(), 0, 1e6f);
        double e = std::fmax(rel_to_row_scale(be.read<float>(dq, q.size()), rq, nq * hd),
                             rel_to_row_scale(be.read<float>(dk, k.size()), rk, nkv * hd));
        expect(e <= TOL, "launch_rope_qk", e);
        auto rn = q;
        orc_qk_norm_rope_rows(rn.data(), wq.data(), T, nq, hd, 1e-6f, hd, pos.data(), 1e6f, 1.f, ORC_ROPE_NEOX, 1);
        auto dn = be.upload(q);
        auto dwq = be.upload(wq);
        be.launch_qk_norm_rope(dn.as<float>(), dwq.as<float>(), T, nq, hd, 1e-6f, hd, dp.as<int32_t>(), 0, 1e6f);
        e = rel_to_row_scale(be.read<float>(dn, q.size()), rn, nq * hd);
        expect(e <= TOL, "launch_qk_norm_rope", e);
    }
    {  // silu*mul
        auto g = randn(T * I), u = randn(T * I);
        std::vector<float> ref(T * I);
        orc_silu_mul(g.data(), u.data(), ref.data(), T * I, 1);
        auto dg = be.upload(g), du = be.upload(u);
        auto out = be.launch_silu_mul(dg.as<float>(), du.as<float>(), T * I);
        double e = rel_to_row_scale(be.read<float>(out, T * I), ref, I);
        expect(e <= TOL, "launch_silu_mul", e);
    }
    {  // causal softmax
        const int64_t L = 256, R = 2 * L;
        auto s = randn(R * L);
        for (auto &x : s) x *= 2.f;
        std::vector<int32_t> nv(R);
        for (int64_t r = 0; r < R; r++) nv[r] = (int32_t)(r % L) + 1;
        std::vector<float> ref(R * L);
        orc_softmax_rows(s.data(), ref.data(), R, L, L, nv.data(), 1);
        auto ds = be.upload(s);
        auto out = be.launch_softmax_rows(ds.as<float>(), R, L, nullptr, (int)L, 0);
        double e = rel_to_row_scale(be.read<float>(out, R * L), ref, L);
        expect(e <= TOL, "launch_softmax_rows", e);
    }
    {  // softmax that takes the score scale (raw dot products in, 1/sqrt(head_dim) folded in)
        const int64_t L = 384, R = 64;
        auto s = randn(R * L);
        const float scale = 1.0f / std::sqrt(128.0f);
        std::vector<float> scaled(s.size()), ref(R * L);
        for (size_t i = 0; i < s.size(); i++) { s[i] *= 22.f; scaled[i] = s[i] * scale; }
        orc_softmax_rows(scaled.data(), ref.data(), R, L, L, nullptr, 1);
        auto ds = be.upload(s);
        auto out = be.empty(4 * R * L);
        be.launch_softmax_rows_scaled(ds.as<float>(), out.as<float>(), nullptr, R, L, L, nullptr, 0, 0, scale);
        double e = rel_to_row_scale(be.read<float>(out, R * L), ref, L);
        expect(e <= TOL, "launch_softmax_rows_scaled", e);
    }
    {  // residual add + norm with the normed row stored as f16: the f32 result, rounded
        auto x = randn(T * H), d = randn(T * H), w = weight(H);
        auto dx = be.upload(x), dd = be.upload(d), dw = be.upload(w);
        auto f32pair = be.launch_add_residual_rms_norm(dx.as<float>(), dd.as<float>(), dw.as<float>(), T, H, 1e-6f);
        auto h16pair = be.launch_add_residual_rms_norm_out16(dx.as<float>(), dd.as<float>(), dw.as<float>(), T, H, 1e-6f, AGN_F16);
        auto n32 = be.read<float>(f32pair.second, T * H);
        auto n16 = be.read<uint16_t>(h16pair.second, T * H);
        auto x32 = be.read<float>(f32pair.first, T * H), x32b = be.read<float>(h16pair.first, T * H);
        // decode the halves exactly and compare with the f32 result: half an f16 ulp at most
        double worst = 0.0;
        for (size_t i = 0; i < n32.size(); i++) {
            const double v = (double)orc_f16_to_f32(n16[i]);
            worst = std::fmax(worst, std::fabs(v - (double)n32[i]) / std::fmax(std::fabs((double)n32[i]), 6.2e-5));
        }
        expect(worst <= 4.9e-4 && std::memcmp(x32.data(), x32b.data(), x32.size() * 4) == 0, "add_residual_rms_norm_out16", worst);
    }
    for (int dtype : {AGN_Q8_0, AGN_Q4_K, AGN_Q6_K}) {  // get_rows, bit-exact
        const size_t rb = agn_type_size(dtype, H);
        std::vector<uint8_t> table(vocab * rb);
        for (auto &b : table) b = (uint8_t)(rng() & 0xff);
        // keep the f16 scales finite: clear the top exponent bit of every 16-bit word that is a scale
        const size_t bb = dtype == AGN_Q8_0 ? 34 : dtype == AGN_Q4_K ? 144 : 210;
        for (size_t off = 0; off + bb <= table.size(); off += bb) {
            if (dtype == AGN_Q8_0) table[off + 1] &= 0x3f;
            if (dtype == AGN_Q4_K) { table[off + 1] &= 0x3f; table[off + 3] &= 0x3f; }
            if (dtype == AGN_Q6_K) table[off + 209] &= 0x3f;
        }
        std::vector<uint32_t> ids(T);
        for (auto &i : ids) i = rng() % vocab;
        std::vector<float> ref(T * H);
        int rc = orc_get_rows(dtype, table.data(), table.size(), vocab, H, ids.data(), T, ref.data(), 1);
        auto dt = be.upload(table);
        auto di = be.upload(ids);
        auto out = be.get_rows(dtype, dt.ptr(), table.size(), vocab, H, di.as<uint32_t>(), T);
        auto got = be.read<float>(out, T * H);
        expect(rc == ORC_OK && std::memcmp(got.data(), ref.data(), got.size() * sizeof(float)) == 0,
               dtype == AGN_Q8_0 ? "get_rows Q8_0 (bit-exact)" : dtype == AGN_Q4_K ? "get_rows Q4_K (bit-exact)" : "get_rows Q6_K (bit-exact)");
        if (dtype == AGN_Q8_0) {
            bool threw = false;
            try { be.dequant_row(dtype, dt.ptr(), table.size(), vocab, H, (uint32_t)vocab); }
            catch (const agn::BackendError &e) { threw = e.status == AGN_EOOB_ID; }
            expect(threw, "dequant_row out of range");
        }
    }
    {  // a GGUF container parsed from memory: one metadata value, one F32 tensor, uploaded and read back through get_rows
        std::vector<uint8_t> blob;
        auto put = [&](const void *p, size_t n) { const uint8_t *b = (const uint8_t *)p; blob.insert(blob.end(), b, b + n); };
        auto put_u32 = [&](uint32_t v) { put(&v, 4); };
        auto put_u64 = [&](uint64_t v) { put(&v, 8); };
        auto put_str = [&](const char *s) { put_u64(std::strlen(s)); put(s, std::strlen(s)); };
        put("GGUF", 4); put_u32(3); put_u64(1); put_u64(1);           // magic, version, 1 tensor, 1 key
        put_str("llama.embedding_length"); put_u32(4); put_u32(8);     // u32 value 8
        put_str("w"); put_u32(2); put_u64(8); put_u64(3); put_u32(0); put_u64(0);  // tensor "w": dims [8, 3], F32, offset 0
        while (blob.size() % 32) blob.push_back(0);                    // data section alignment
        std::vector<float> w(24);
        for (int i = 0; i < 24; i++) w[i] = 0.5f * (float)i - 3.f;
        put(w.data(), w.size() * 4);
        agn::GgufFile g(blob.data(), blob.size());
        uint64_t h = 0;
        agn_tensor_info ti;
        auto table = g.upload(be, "w", &ti);
        const uint32_t ids_h[2] = {2, 0};
        auto di = be.upload(std::vector<uint32_t>(ids_h, ids_h + 2));
        auto rows = be.read<float>(be.get_rows(ti.ggml_type, table.ptr(), (size_t)ti.n_bytes, (int64_t)ti.n_rows, (int64_t)ti.row_len,
                                               di.as<uint32_t>(), 2), 16);
        bool same = g.get_u64("llama.embedding_length", &h) && h == 8 && g.version() == 3 && ti.n_rows == 3 && ti.row_len == 8;
        for (int i = 0; i < 8; i++) same = same && rows[i] == w[16 + i] && rows[8 + i] == w[i];
        expect(same, "GgufFile parse + upload + get_rows");
        // the pre-upload loop on the same container (memory of the caller: no pages to release)
        std::vector<agn_tensor_info> infos;
        uint64_t released = 1;
        auto all = g.upload_all(be, {"w"}, true, &infos, &released);
        auto back = be.read<float>(all[0], w.size());
        expect(all.size() == 1 && infos[0].n_bytes == w.size() * 4 && released == 0 && back == w, "GgufFile upload_all");
    }
    {  // softmax that writes the valid entries only: the tail keeps the sentinel, the valid part matches the oracle
        const int R = 5, L = 516;
        std::vector<float> sc(R * L), ref(R * L, 0.f), sentinel(R * L, -7.25f);
        for (auto &v : sc) v = 2.f * N01(rng);
        std::vector<int32_t> nv = {L, 1, 300, 0, 515};
        orc_softmax_rows(sc.data(), ref.data(), R, L, L, nv.data(), 1);
        auto ds = be.upload(sc);
        auto dn = be.upload(nv);
        auto dout = be.upload(sentinel);
        be.launch_softmax_rows_valid(ds.as<float>(), dout.ptr(), nullptr, R, L, L, dn.as<int32_t>(), 0, 0, 1.0f, AGN_F32);
        auto got = be.read<float>(dout, R * L);
        double worst = 0;
        bool tail_kept = true;
        for (int r = 0; r < R; r++) {
            float scale = 1e-30f;
            for (int i = 0; i < nv[r]; i++) scale = std::fmax(scale, std::fabs(ref[r * L + i]));
            for (int i = 0; i < L; i++) {
                if (i < nv[r]) worst = std::fmax(worst, std::fabs((double)got[r * L + i] - ref[r * L + i]) / scale);
                else tail_kept = tail_kept && got[r * L + i] == -7.25f;
            }
        }
        expect(worst <= 1e-5 && tail_kept && !be.last_kernel().empty(), "softmax_rows_valid", worst);
    }
    {  // Q8_K activation rows: the standalone quantiser is the oracle's bytes; the fused norm agrees with the two launches
        const int T = 9, H = 1024, nb = H / 256;
        auto x = randn((size_t)T * H), w = weight(H);
        x[5] = 3.0f; x[9] = -3.0f;  // a tie in magnitude inside the first block
        std::vector<float> rd((size_t)T * nb);
        std::vector<int8_t> rq((size_t)T * H);
        std::vector<int16_t> rb((size_t)T * nb * 16);
        orc_quantize_rows_q8_k(x.data(), T, H, rd.data(), rq.data(), rb.data(), 1);
        auto dx = be.upload(x), dw = be.upload(w);
        auto q = be.launch_quantize_rows_q8_k(dx.as<float>(), T, H);
        bool same = be.read<float>(q.d, rd.size()) == rd && be.read<int8_t>(q.qs, rq.size()) == rq &&
                    be.read<int16_t>(q.bsums, rb.size()) == rb;
        expect(same, "launch_quantize_rows_q8_k bit-exact");
        auto normed = be.launch_rms_norm(dx.as<float>(), dw.as<float>(), T, H, 1e-6f);
        auto two = be.launch_quantize_rows_q8_k(normed.as<float>(), T, H);
        auto fused = be.launch_rms_norm_q8_k(dx.as<float>(), dw.as<float>(), T, H, 1e-6f);
        // (the fused kernel adds the squares in another order: the scale factor may differ in the last bit)
        auto d2 = be.read<float>(two.d, rd.size()), df = be.read<float>(fused.d, rd.size());
        auto q2 = be.read<int8_t>(two.qs, rq.size()), qf = be.read<int8_t>(fused.qs, rq.size());
        same = true;
        for (size_t i = 0; i < d2.size(); i++) same = same && std::fabs(d2[i] - df[i]) <= 1e-5f * std::fabs(d2[i]);
        size_t off = 0;
        for (size_t i = 0; i < q2.size(); i++) {
            same = same && std::abs((int)q2[i] - (int)qf[i]) <= 1;
            off += q2[i] != qf[i];
        }
        same = same && off * 500 < q2.size();
        expect(same, "launch_rms_norm_q8_k against rms_norm then quantize");
    }
    {  // error behaviour: bad argument -> status + message, context still usable
        bool threw = false;
        auto d = be.empty(512);
        try { be.launch_rope(d.as<float>(), 1, 1, 128, 130, nullptr, 0, 1e4f); }
        catch (const agn::BackendError &e) { threw = e.status == AGN_EINVAL && std::strstr(e.what(), "n_rot") != nullptr; }
        expect(threw, "EINVAL on n_rot > head_dim");
        be.sync();
    }
    std::printf("kernels launched: %llu, failures: %d\n", (unsigned long long)be.launch_count(), failures);
    return failures ? 1 : 0;
}
