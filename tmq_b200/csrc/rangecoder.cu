// Host-side entropy coding of packed ternary matrices: byte-compatible with the streams the reference writes into
// state dicts (framing tmq/tmq_native.cpp:50-140, coder tmq/rangecoder.h:41-193, bit writer tmq/bitstream.h:31-177).
//
// Stream = 26-byte big-endian header { u64 symbol count, u64 payload bits, u32 total bytes, 3 x u16 frequencies of
// (-1, 0, +1) scaled to 65535 } + payload of a carry-less 32-bit range coder with byte-wise renormalisation + one
// spare zero byte.  Symbols are visited row by row over the PACKED matrix P[rows][ceil(cols/16)], pad elements of
// the last word of a row skipped.  Inherently sequential, so it runs on the host; nothing here touches the GPU.
#include <stdint.h>
#include <string.h>

#include <vector>

#include "tmq_b200.h"

namespace {

constexpr size_t kHeader = 26;

struct Model {
    uint32_t freq[3];
    uint32_t cum[3];
    uint32_t total;
    void set(const uint16_t f[3]) {
        for (int i = 0; i < 3; i++) freq[i] = f[i];
        cum[0] = 0;
        cum[1] = freq[0];
        cum[2] = freq[0] + freq[1];
        total = cum[2] + freq[2];
    }
};

inline uint32_t symbol_of_code(uint32_t code) { return code == 0u ? 1u : (code == 1u ? 2u : (code == 2u ? 0u : 3u)); }
inline uint32_t code_of_symbol(uint32_t s) { return s == 0u ? 2u : (s == 1u ? 0u : 1u); }

template <typename F>
inline void for_each_code(const uint32_t *P, int64_t rows, int64_t cols, F &&fn) {
    const int64_t Q = (cols + 15) / 16;
    for (int64_t r = 0; r < rows; r++) {
        for (int64_t q = 0; q < Q; q++) {
            const uint32_t w = P[r * Q + q];
            const int lim = (int)((cols - q * 16 < 16) ? (cols - q * 16) : 16);
            for (int i = 0; i < lim; i++) fn((w >> (30 - 2 * i)) & 3u);
        }
    }
}

void put_be(uint8_t *p, uint64_t v, int bytes) {
    for (int i = 0; i < bytes; i++) p[i] = (uint8_t)(v >> (8 * (bytes - 1 - i)));
}
uint64_t get_be(const uint8_t *p, int bytes) {
    uint64_t v = 0;
    for (int i = 0; i < bytes; i++) v = (v << 8) | p[i];
    return v;
}

struct Encoder {
    uint32_t low = 0, range = 0xFFFFFFFFu;
    std::vector<uint8_t> &out;
    explicit Encoder(std::vector<uint8_t> &o) : out(o) {}
    void put(uint32_t s, const Model &m) {
        range /= m.total;
        low += m.cum[s] * range;
        range *= m.freq[s];
        for (;;) {
            const bool top_settled = ((low ^ (low + range)) < (1u << 24));
            if (!top_settled) {
                if (range >= (1u << 16)) break;
                range = (0u - low) & 0xFFFFu;  // underflow: shrink the interval to what fits below the carry
            }
            out.push_back((uint8_t)(low >> 24));
            low <<= 8;
            range <<= 8;
        }
    }
    void finish() {
        for (int i = 0; i < 4; i++) {
            out.push_back((uint8_t)(low >> 24));
            low <<= 8;
        }
    }
};

struct Decoder {
    uint32_t low = 0, range = 0xFFFFFFFFu, window = 0;
    const uint8_t *p;
    size_t n, pos = 0;
    Decoder(const uint8_t *data, size_t bytes) : p(data), n(bytes) {
        for (int i = 0; i < 4; i++) window = (window << 8) | next();
    }
    uint8_t next() { return pos < n ? p[pos++] : (uint8_t)0; }
    uint32_t get(const Model &m) {
        range /= m.total;
        const uint32_t f = (window - low) / range;
        // same bisection over the cumulative table as the reference (tmq/rangecoder.h:170-180)
        int lo = 0, hi = 3, s;
        for (;;) {
            const int mid = (lo + hi) / 2;
            if (m.cum[mid] > f) { hi = mid; continue; }
            if (mid >= 2 || m.cum[mid + 1] > f) { s = mid; break; }
            lo = mid;
        }
        low += m.cum[s] * range;
        range *= m.freq[s];
        for (;;) {
            if ((low ^ (low + range)) >= (1u << 24)) {
                if (range >= (1u << 16)) break;
                range = (0u - low) & 0xFFFFu;
            }
            window = (window << 8) | next();
            low <<= 8;
            range <<= 8;
        }
        return (uint32_t)s;
    }
};

}  // namespace

extern "C" size_t tmq_rc_encode_bound(int64_t rows, int64_t cols) {
    if (rows <= 0 || cols <= 0) return kHeader + 8;
    // worst case of a 3-symbol model with 16-bit frequencies is < 17 bits per symbol; plus header, flush, spare
    return kHeader + 16 + (size_t)(((unsigned long long)rows * (unsigned long long)cols * 17ull + 7ull) / 8ull);
}

extern "C" int tmq_rc_encode(const uint32_t *P, int64_t rows, int64_t cols, uint8_t *out, size_t out_cap,
                             size_t *out_len) {
    if (!P || !out || !out_len || rows <= 0 || cols <= 0) return TMQ_ERR_ARG;
    uint64_t hist[4] = {0, 0, 0, 0};
    for_each_code(P, rows, cols, [&](uint32_t c) { hist[symbol_of_code(c)]++; });
    if (hist[3] != 0) return TMQ_ERR_ARG;  // code 11 is not a ternary value
    const uint64_t total = hist[0] + hist[1] + hist[2];
    const float scale = 65535.f / (float)total;
    uint16_t f16[3];
    for (int i = 0; i < 3; i++) f16[i] = (uint16_t)((float)hist[i] * scale);
    for (int i = 0; i < 3; i++)
        if (hist[i] != 0 && f16[i] == 0) return TMQ_ERR_UNSUPPORTED;  // a symbol too rare for a 16-bit model
    Model m;
    m.set(f16);
    std::vector<uint8_t> payload;
    payload.reserve((size_t)(total / 4) + 64);
    Encoder enc(payload);
    for_each_code(P, rows, cols, [&](uint32_t c) { enc.put(symbol_of_code(c), m); });
    enc.finish();
    const uint64_t bits = (uint64_t)payload.size() * 8u;
    payload.push_back(0);  // the reference's bit writer always carries one spare zero byte
    const size_t need = kHeader + payload.size();
    if (need > 0xFFFFFFFFull) return TMQ_ERR_UNSUPPORTED;
    if (need > out_cap) return TMQ_ERR_SCRATCH;
    put_be(out, (uint64_t)rows * (uint64_t)cols, 8);
    put_be(out + 8, bits, 8);
    put_be(out + 16, need, 4);
    for (int i = 0; i < 3; i++) put_be(out + 20 + 2 * i, f16[i], 2);
    memcpy(out + kHeader, payload.data(), payload.size());
    *out_len = need;
    return TMQ_OK;
}

extern "C" int tmq_rc_decode(const uint8_t *in, size_t in_len, uint32_t *P, int64_t rows, int64_t cols) {
    if (!in || !P || rows <= 0 || cols <= 0 || in_len < kHeader) return TMQ_ERR_ARG;
    const uint64_t nsym = get_be(in, 8);
    if (nsym == 0) {
        P[0] = 0;
        return TMQ_ERR_ARG;  // an empty stream cannot fill a matrix (the reference rejects it too)
    }
    const uint64_t bits = get_be(in + 8, 8);
    if (get_be(in + 16, 4) < kHeader) return TMQ_ERR_ARG;
    uint16_t f16[3];
    for (int i = 0; i < 3; i++) f16[i] = (uint16_t)get_be(in + 20 + 2 * i, 2);
    Model m;
    m.set(f16);
    if (m.total == 0) return TMQ_ERR_ARG;
    size_t nbytes = (size_t)((bits + 7) / 8);
    if (nbytes > in_len - kHeader) nbytes = in_len - kHeader;
    Decoder dec(in + kHeader, nbytes);
    const int64_t Q = (cols + 15) / 16;
    for (int64_t r = 0; r < rows; r++) {
        for (int64_t q = 0; q < Q; q++) {
            const int lim = (int)((cols - q * 16 < 16) ? (cols - q * 16) : 16);
            uint32_t w = 0;
            for (int i = 0; i < lim; i++) {
                if (dec.range < m.total) return TMQ_ERR_ARG;  // corrupt stream: would divide by zero next
                w = (w << 2) | code_of_symbol(dec.get(m));
            }
            if (lim != 16) w <<= 2 * (16 - lim);
            P[r * Q + q] = w;
        }
    }
    return TMQ_OK;
}
