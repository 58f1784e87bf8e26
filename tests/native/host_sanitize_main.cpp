// Driver for the address / undefined-behaviour sanitizer build of the host runtime library: exercises the
// parallel span reader and the trace recorder from several threads and checks what they return.
#include <fcntl.h>
#include <unistd.h>

#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <thread>
#include <vector>

#include "../../zml_b200/csrc/host/zb_host.h"

#define CHECK(cond)                                                        \
  do {                                                                     \
    if (!(cond)) {                                                         \
      std::fprintf(stderr, "CHECK failed at line %d: %s\n", __LINE__, #cond); \
      return 1;                                                            \
    }                                                                      \
  } while (0)

int main(int argc, char** argv) {
  const std::string dir = argc > 1 ? argv[1] : "/tmp";
  // ---- file streaming: ragged spans, more spans than threads, a zero-length span, a read past the end
  const std::string path = dir + "/zb_sanitize_blob.bin";
  const size_t n = 3u << 20;
  std::vector<unsigned char> blob(n);
  for (size_t i = 0; i < n; ++i) blob[i] = static_cast<unsigned char>((i * 2654435761u) >> 13);
  {
    FILE* f = std::fopen(path.c_str(), "wb");
    CHECK(f != nullptr);
    CHECK(std::fwrite(blob.data(), 1, n, f) == n);
    std::fclose(f);
  }
  const int fd = open(path.c_str(), O_RDONLY);
  CHECK(fd >= 0);
  std::vector<long long> offs, lens;
  long long total = 0;
  for (int i = 0; i < 37; ++i) {
    const long long off = (static_cast<long long>(i) * 80021) % static_cast<long long>(n - 70000);
    const long long len = i == 5 ? 0 : 1 + (i * 7919) % 65536;
    offs.push_back(off);
    lens.push_back(len);
    total += len;
  }
  for (int threads : {1, 3, 8, 64}) {
    std::vector<unsigned char> dst(static_cast<size_t>(total) + 1, 0xAB);
    const long long got = zbh_pread_spans(fd, offs.data(), lens.data(), static_cast<int>(offs.size()), dst.data(), threads);
    CHECK(got == total);
    size_t at = 0;
    for (size_t i = 0; i < offs.size(); ++i) {
      CHECK(std::memcmp(dst.data() + at, blob.data() + offs[i], static_cast<size_t>(lens[i])) == 0);
      at += static_cast<size_t>(lens[i]);
    }
    CHECK(dst[static_cast<size_t>(total)] == 0xAB);      // nothing written past the requested bytes
  }
  {
    long long off = static_cast<long long>(n) - 10, len = 100;      // crosses the end of the file
    std::vector<unsigned char> dst(128, 0);
    const long long got = zbh_pread_spans(fd, &off, &len, 1, dst.data(), 2);
    CHECK(got < 100);                                            // short read or error, never an overrun
  }
  close(fd);
  std::remove(path.c_str());

  // ---- tracer: spans from several threads, ring overflow, JSON dump, restart
  CHECK(zbh_trace_start(256) == 0);
  std::vector<std::thread> workers;
  for (int t = 0; t < 6; ++t) {
    workers.emplace_back([t] {
      for (int i = 0; i < 200; ++i) {
        const std::string name = "worker" + std::to_string(t) + "#i=" + std::to_string(i) + "#";
        const unsigned long long outer = zbh_trace_begin(name.c_str());
        const unsigned long long inner = zbh_trace_begin("inner");
        zbh_trace_instant("tick");
        zbh_trace_end(inner);
        zbh_trace_end(outer);
      }
    });
  }
  for (auto& w : workers) w.join();
  CHECK(zbh_trace_count() > 0);
  zbh_trace_end(123456789ull);                                     // unknown span id: ignored
  const std::string json = dir + "/zb_sanitize_trace.json";
  CHECK(zbh_trace_write_json(json.c_str()) == 0);
  {
    FILE* f = std::fopen(json.c_str(), "rb");
    CHECK(f != nullptr);
    char head[2] = {0, 0};
    CHECK(std::fread(head, 1, 1, f) == 1);
    CHECK(head[0] == '{' || head[0] == '[');
    std::fclose(f);
  }
  std::remove(json.c_str());
  CHECK(zbh_trace_stop() == 0);
  CHECK(zbh_trace_start(16) == 0);
  zbh_trace_end(zbh_trace_begin("again"));
  CHECK(zbh_trace_stop() == 0);
  std::puts("HOST_SANITIZE_OK");
  return 0;
}
