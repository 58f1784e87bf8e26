// Host span tracer.  The reference wraps TSL's TraceMe recorder and NVTX push/pop
// (zml/profiling/traceme_lib.cc:61-252) and converts the recorded XSpace to trace
// events; here spans go into a lock-free-ish ring (one mutex per push, off the hot
// device path) and are written directly as Chrome / Perfetto trace-event JSON.
// NVTX ranges are emitted through dlopen'ed libnvToolsExt when it is present, so
// external profilers see the same span names.
#include <dlfcn.h>
#include <stdio.h>
#include <string.h>
#include <time.h>
#include <unistd.h>

#include <atomic>
#include <mutex>
#include <string>
#include <thread>
#include <vector>

#include "zb_host.h"

namespace {
struct Event {
  std::string name;
  unsigned long long id;
  long long ts_ns;
  long long dur_ns;   // -1: still open, -2: instant
  unsigned long long tid;
};

std::mutex g_mu;
std::vector<Event> g_events;
size_t g_capacity = 0;
std::atomic<bool> g_on{false};
std::atomic<unsigned long long> g_next_id{1};
long long g_dropped = 0;

typedef int (*nvtx_push_t)(const char*);
typedef int (*nvtx_pop_t)(void);
nvtx_push_t g_nvtx_push = nullptr;
nvtx_pop_t g_nvtx_pop = nullptr;
std::once_flag g_nvtx_once;

void load_nvtx() {
  std::call_once(g_nvtx_once, [] {
    const char* names[] = {"libnvToolsExt.so.1", "libnvToolsExt.so"};
    for (const char* n : names) {
      void* h = dlopen(n, RTLD_NOW | RTLD_LOCAL);
      if (h) {
        g_nvtx_push = reinterpret_cast<nvtx_push_t>(dlsym(h, "nvtxRangePushA"));
        g_nvtx_pop = reinterpret_cast<nvtx_pop_t>(dlsym(h, "nvtxRangePop"));
        if (g_nvtx_push && g_nvtx_pop) return;
      }
    }
  });
}

long long now_ns() {
  timespec ts;
  clock_gettime(CLOCK_MONOTONIC, &ts);
  return static_cast<long long>(ts.tv_sec) * 1000000000ll + ts.tv_nsec;
}

unsigned long long tid() {
  return static_cast<unsigned long long>(std::hash<std::thread::id>()(std::this_thread::get_id()) & 0xffffff);
}

void json_escape(FILE* f, const std::string& s) {
  for (char c : s) {
    if (c == '"' || c == '\\') {
      fputc('\\', f);
      fputc(c, f);
    } else if (static_cast<unsigned char>(c) < 0x20) {
      fprintf(f, "\\u%04x", c);
    } else {
      fputc(c, f);
    }
  }
}
}  // namespace

extern "C" {

int zbh_trace_start(size_t capacity_events) {
  std::lock_guard<std::mutex> l(g_mu);
  g_events.clear();
  g_capacity = capacity_events ? capacity_events : (1u << 20);
  g_events.reserve(g_capacity < 65536 ? g_capacity : 65536);
  g_dropped = 0;
  load_nvtx();
  g_on.store(true);
  return 0;
}

int zbh_trace_stop(void) {
  g_on.store(false);
  return 0;
}

unsigned long long zbh_trace_begin(const char* name) {
  if (g_nvtx_push) g_nvtx_push(name);
  if (!g_on.load()) return 0;
  const unsigned long long id = g_next_id.fetch_add(1);
  std::lock_guard<std::mutex> l(g_mu);
  if (g_events.size() >= g_capacity) {
    ++g_dropped;
    return 0;
  }
  g_events.push_back({name, id, now_ns(), -1, tid()});
  return id;
}

void zbh_trace_end(unsigned long long span_id) {
  if (g_nvtx_pop) g_nvtx_pop();
  if (span_id == 0) return;
  const long long t = now_ns();
  std::lock_guard<std::mutex> l(g_mu);
  for (size_t i = g_events.size(); i-- > 0;) {
    if (g_events[i].id == span_id) {
      g_events[i].dur_ns = t - g_events[i].ts_ns;
      return;
    }
  }
}

void zbh_trace_instant(const char* name) {
  if (!g_on.load()) return;
  std::lock_guard<std::mutex> l(g_mu);
  if (g_events.size() >= g_capacity) {
    ++g_dropped;
    return;
  }
  g_events.push_back({name, g_next_id.fetch_add(1), now_ns(), -2, tid()});
}

long long zbh_trace_count(void) {
  std::lock_guard<std::mutex> l(g_mu);
  return static_cast<long long>(g_events.size());
}

// Span names follow the reference's encoding `name#k=v,k=v#` (zml/profiling/tracer.zig:41-102);
// the metadata part is split out into the event's "args".
int zbh_trace_write_json(const char* path) {
  std::lock_guard<std::mutex> l(g_mu);
  FILE* f = fopen(path, "w");
  if (!f) return -1;
  fprintf(f, "{\"displayTimeUnit\":\"ns\",\"traceEvents\":[\n");
  const int pid = static_cast<int>(getpid());
  bool first = true;
  for (const Event& e : g_events) {
    std::string name = e.name, meta;
    const size_t h = name.find('#');
    if (h != std::string::npos) {
      meta = name.substr(h + 1);
      if (!meta.empty() && meta.back() == '#') meta.pop_back();
      name = name.substr(0, h);
    }
    if (!first) fprintf(f, ",\n");
    first = false;
    fprintf(f, "{\"name\":\"");
    json_escape(f, name);
    if (e.dur_ns == -2) {
      fprintf(f, "\",\"ph\":\"i\",\"s\":\"t\",\"ts\":%.3f", e.ts_ns / 1000.0);
    } else {
      const long long d = e.dur_ns < 0 ? 0 : e.dur_ns;
      fprintf(f, "\",\"ph\":\"X\",\"ts\":%.3f,\"dur\":%.3f", e.ts_ns / 1000.0, d / 1000.0);
    }
    fprintf(f, ",\"pid\":%d,\"tid\":%llu,\"args\":{", pid, e.tid);
    bool firsta = true;
    size_t pos = 0;
    while (pos < meta.size()) {
      size_t comma = meta.find(',', pos);
      if (comma == std::string::npos) comma = meta.size();
      const std::string kv = meta.substr(pos, comma - pos);
      const size_t eq = kv.find('=');
      if (eq != std::string::npos) {
        if (!firsta) fputc(',', f);
        firsta = false;
        fputc('"', f);
        json_escape(f, kv.substr(0, eq));
        fprintf(f, "\":\"");
        json_escape(f, kv.substr(eq + 1));
        fputc('"', f);
      }
      pos = comma + 1;
    }
    fprintf(f, "}}");
  }
  fprintf(f, "\n],\"droppedEvents\":%lld}\n", g_dropped);
  fclose(f);
  return 0;
}

}  // extern "C"
