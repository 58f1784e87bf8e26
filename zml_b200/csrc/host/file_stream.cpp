// Parallel positional reads for the weight loader: a tensor shard is a list of byte
// ranges of a safetensors file; they are read with pread(2) from several threads
// straight into the (pinned) destination buffer, so the host->device copy can start
// as soon as the call returns.  Plays the role of the reference's DirectMemoryWriter
// file side (zml/io.zig:656-825).
#include <errno.h>
#include <unistd.h>

#include <algorithm>
#include <atomic>
#include <thread>
#include <vector>

#include "zb_host.h"

namespace {
struct Piece {
  long long file_off;
  long long len;
  long long dst_off;
};

long long read_piece(int fd, const Piece& p, char* dst) {
  long long done = 0;
  while (done < p.len) {
    ssize_t r = pread(fd, dst + p.dst_off + done, static_cast<size_t>(p.len - done), p.file_off + done);
    if (r < 0) {
      if (errno == EINTR) continue;
      return -static_cast<long long>(errno);
    }
    if (r == 0) return -static_cast<long long>(EIO);   // unexpected end of file
    done += r;
  }
  return done;
}
}  // namespace

extern "C" long long zbh_pread_spans(int fd, const long long* offsets, const long long* lengths, int n,
                                     void* dst, int threads) {
  if (n <= 0) return 0;
  // cut large ranges into 8 MiB pieces so that threads share one big range too
  constexpr long long kPiece = 8ll << 20;
  std::vector<Piece> pieces;
  long long dst_off = 0;
  for (int i = 0; i < n; ++i) {
    long long off = offsets[i], left = lengths[i];
    while (left > 0) {
      const long long l = std::min(left, kPiece);
      pieces.push_back({off, l, dst_off});
      off += l;
      dst_off += l;
      left -= l;
    }
  }
  const int nt = std::max(1, std::min<int>(threads, static_cast<int>(pieces.size())));
  std::atomic<size_t> next{0};
  std::atomic<long long> err{0};
  std::atomic<long long> total{0};
  auto work = [&] {
    while (true) {
      const size_t i = next.fetch_add(1);
      if (i >= pieces.size() || err.load() != 0) return;
      const long long r = read_piece(fd, pieces[i], static_cast<char*>(dst));
      if (r < 0) {
        err.store(r);
        return;
      }
      total.fetch_add(r);
    }
  };
  if (nt == 1) {
    work();
  } else {
    std::vector<std::thread> pool;
    for (int t = 0; t < nt; ++t) pool.emplace_back(work);
    for (auto& th : pool) th.join();
  }
  return err.load() != 0 ? err.load() : total.load();
}
