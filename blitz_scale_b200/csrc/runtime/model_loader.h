// Disk -> host loader for flat weight-segment files: O_DIRECT reads in large chunks from several
// threads into a caller-provided (pinned, page-aligned) buffer, the ServerlessLLM-style baseline
// path (src/blitz/model_loader.cc:40-116: O_DIRECT + 2 threads x 64 MB pread).  The host buffer
// doubles as the host cache for LOAD_FROM_HOST_MEM; host -> device copies are issued by the engine
// in chunks on two streams (src/blitz/model_loader.cc:244-295).
#pragma once
#include <pybind11/pybind11.h>
#include <fcntl.h>
#include <sys/stat.h>
#include <unistd.h>
#include <atomic>
#include <chrono>
#include <cstdint>
#include <cstring>
#include <stdexcept>
#include <string>
#include <thread>
#include <vector>

#include "../util/log.h"

namespace blitz {

struct LoadResult {
  int64_t bytes = 0;
  double seconds = 0;
  bool direct_io = false;
};

inline LoadResult load_file_to_host(const std::string& path, uintptr_t dst_addr, int64_t expect_bytes, int threads = 2,
                                    int64_t chunk = 64ll << 20) {
  struct stat st;
  if (stat(path.c_str(), &st) != 0) throw std::runtime_error("cannot stat " + path);
  if (expect_bytes >= 0 && st.st_size != expect_bytes)
    throw std::runtime_error("segment file size " + std::to_string(st.st_size) + " != expected " + std::to_string(expect_bytes));
  const int64_t total = st.st_size;
  char* dst = reinterpret_cast<char*>(dst_addr);
  bool direct = (dst_addr % 4096 == 0);
  int fd = direct ? open(path.c_str(), O_RDONLY | O_DIRECT) : -1;
  if (fd < 0) {
    direct = false;
    fd = open(path.c_str(), O_RDONLY);
  }
  if (fd < 0) throw std::runtime_error("cannot open " + path);
  auto t0 = std::chrono::steady_clock::now();
  std::atomic<int64_t> next{0};
  std::atomic<bool> failed{false};
  auto work = [&] {
    while (!failed.load()) {
      const int64_t off = next.fetch_add(chunk);
      if (off >= total) break;
      int64_t len = std::min<int64_t>(chunk, total - off);
      int64_t done = 0;
      while (done < len) {
        // O_DIRECT wants sector-multiple lengths; the ragged tail is read through a buffered descriptor below
        int64_t want = len - done;
        if (direct && (want % 4096) != 0) want -= want % 4096;
        if (want == 0) break;
        ssize_t r = pread(fd, dst + off + done, static_cast<size_t>(want), off + done);
        if (r <= 0) { failed = true; return; }
        done += r;
      }
      if (done < len) {
        int fd2 = open(path.c_str(), O_RDONLY);
        if (fd2 < 0) { failed = true; return; }
        while (done < len) {
          ssize_t r = pread(fd2, dst + off + done, static_cast<size_t>(len - done), off + done);
          if (r <= 0) { failed = true; break; }
          done += r;
        }
        close(fd2);
      }
    }
  };
  std::vector<std::thread> pool;
  for (int i = 0; i < std::max(1, threads); ++i) pool.emplace_back(work);
  for (auto& t : pool) t.join();
  close(fd);
  if (failed) throw std::runtime_error("read failed: " + path);
  LoadResult res;
  res.bytes = total;
  res.seconds = std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
  res.direct_io = direct;
  BZ_DEBUG("loaded %s: %.3f GB in %.3f s (%.2f GB/s, %s, %d threads)", path.c_str(), total / 1e9, res.seconds,
           total / 1e9 / (res.seconds > 0 ? res.seconds : 1e-9), direct ? "O_DIRECT" : "buffered", threads);
  return res;
}

inline void bind_loader(pybind11::module_& m) {
  namespace py = pybind11;
  py::class_<LoadResult>(m, "LoadResult").def_readonly("bytes", &LoadResult::bytes)
      .def_readonly("seconds", &LoadResult::seconds).def_readonly("direct_io", &LoadResult::direct_io);
  m.def("load_file_to_host", &load_file_to_host, py::arg("path"), py::arg("dst_addr"), py::arg("expect_bytes") = -1,
        py::arg("threads") = 2, py::arg("chunk") = 64ll << 20, py::call_guard<py::gil_scoped_release>());
}

}  // namespace blitz
using blitz::bind_loader;
