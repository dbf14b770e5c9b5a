// Randomised driver for the native host runtime, meant to be compiled together with csrc/host_runtime.cpp under the
// address and undefined-behaviour sanitizers (tests/test_host_runtime.py does that): random vocabularies (with missing
// bytes and an empty entry), random documents through the single and the batch encoder with several thread counts, an
// output buffer that is too small, and the batch gather over every element width with in-range and out-of-range windows.
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <random>
#include <string>
#include <vector>
extern "C" {
void* rk_tok_create(const uint8_t*, const int64_t*, const int32_t*, int32_t);
void rk_tok_free(void*);
int64_t rk_tok_encode(const void*, const uint8_t*, int64_t, int32_t*, int64_t);
int32_t rk_tok_encode_batch(const void*, const uint8_t*, const int64_t*, int64_t, int32_t*, const int64_t*, int64_t*, int32_t);
int32_t rk_gather_rows(const void*, int32_t, int32_t, int64_t, const int64_t*, int64_t, int64_t, int32_t*, int32_t*, int32_t);
}
int main() {
  std::mt19937_64 rng(1);
  for (int round = 0; round < 200; ++round) {
    // random vocabulary: all single bytes + random multi-byte strings
    std::vector<std::string> toks;
    for (int b = 0; b < 256; ++b) if (round % 3 || (b % 7)) toks.push_back(std::string(1, char(b)));
    int extra = rng() % 300;
    for (int i = 0; i < extra; ++i) { std::string s; int len = 1 + rng() % 9; for (int j = 0; j < len; ++j) s.push_back(char('a' + rng() % 4)); toks.push_back(s); }
    if (round % 11 == 0) toks.push_back("");
    std::vector<uint8_t> blob; std::vector<int64_t> off{0}; std::vector<int32_t> ids;
    for (size_t i = 0; i < toks.size(); ++i) { blob.insert(blob.end(), toks[i].begin(), toks[i].end()); off.push_back((int64_t)blob.size()); ids.push_back((int32_t)i + 1); }
    if (blob.empty()) blob.push_back(0);
    void* h = rk_tok_create(blob.data(), off.data(), ids.data(), (int32_t)toks.size());
    if (!h) { printf("create failed\n"); return 1; }
    // documents
    int nd = rng() % 20;
    std::vector<uint8_t> src; std::vector<int64_t> doff{0};
    for (int d = 0; d < nd; ++d) { int len = rng() % 200; for (int j = 0; j < len; ++j) src.push_back(round % 2 ? uint8_t('a' + rng() % 5) : uint8_t(rng())); doff.push_back((int64_t)src.size()); }
    std::vector<int32_t> out(src.size() + 1); std::vector<int64_t> counts(nd + 1);
    if (src.empty()) src.push_back(0);
    rk_tok_encode_batch(h, src.data(), doff.data(), nd, out.data(), doff.data(), counts.data(), (int)(rng() % 5));
    for (int d = 0; d < nd; ++d) {
      int64_t n = doff[d + 1] - doff[d];
      std::vector<int32_t> one(n + 1);
      int64_t c = rk_tok_encode(h, src.data() + doff[d], n, one.data(), n);
      if (c != counts[d]) { printf("mismatch %lld %lld\n", (long long)c, (long long)counts[d]); return 1; }
      // tiny capacity must report overflow, not write past the buffer
      if (n > 2) { std::vector<int32_t> small(1); rk_tok_encode(h, src.data() + doff[d], n, small.data(), 1); }
    }
    rk_tok_free(h);
    // gather
    int64_t total = 50 + rng() % 500; int64_t window = 2 + rng() % 40; if (window > total) window = total;
    int rows = rng() % 12; int es = 1 << (rng() % 4);
    std::vector<uint8_t> stream(total * es); for (auto& x : stream) x = uint8_t(rng());
    std::vector<int64_t> offs(rows + 1);
    for (int r = 0; r < rows; ++r) offs[r] = rng() % (total - window + 1);
    std::vector<int32_t> in((size_t)rows * (window - 1) + 1), tg((size_t)rows * (window - 1) + 1);
    int rc = rk_gather_rows(stream.data(), es, round & 1, total, offs.data(), rows, window, in.data(), tg.data(), (int)(rng() % 4));
    if (rc != 0) { printf("gather rc %d\n", rc); return 1; }
    if (rows) { offs[0] = total - window + 1; if (rk_gather_rows(stream.data(), es, 0, total, offs.data(), rows, window, in.data(), tg.data(), 2) != -2) { printf("bounds not caught\n"); return 1; } }
  }
  printf("fuzz ok\n");
  return 0;
}
