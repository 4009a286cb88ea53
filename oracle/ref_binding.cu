// TEST INFRASTRUCTURE.  Python binding of the REFERENCE's own HetuTable (compiled from the reference's
// sources where they lie, never copied into this repository) under the module name `hetuCTR_ref`.
// Besides the reference's constructor/preprocess/push_pull it exposes `dump`, which copies the reference's
// internal device arrays to numpy so that index parity can be checked bit for bit.  All members of the
// reference class are public (csrc/core/hetu_gpu_table.h:22), so nothing in the reference is modified.
#include <pybind11/numpy.h>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include <cuda_runtime.h>

#include <memory>
#include <string>
#include <algorithm>
#include <chrono>
#include <cstring>
#include <vector>

#include "core/hetu_gpu_table.h"

namespace py = pybind11;
using namespace hetuCTR;

namespace {

template <class T>
py::array_t<long long> fetch(const T *dev, size_t n) {
  std::vector<T> tmp(n);
  if (n) cudaMemcpy(tmp.data(), dev, n * sizeof(T), cudaMemcpyDeviceToHost);
  py::array_t<long long> out(n);
  auto o = out.mutable_data();
  for (size_t i = 0; i < n; i++) o[i] = (long long)tmp[i];
  return out;
}

py::array dump(HetuTable &t, const std::string &what, bool prev) {
  cudaSetDevice(t.device_id_);
  cudaDeviceSynchronize();
  PreprocessData &b = prev ? t.prev_batch_ : t.cur_batch_;
  const size_t B = b.batch_size, U = b.unique_size, n = t.nrank_;
  if (what == "unique_idx") return fetch(b.d_unique_idx, U);
  if (what == "idx_map") return fetch(b.d_idx_map, B);
  if (what == "sorted_arg") return fetch(b.d_sorted_arg, B);
  if (what == "run_length") return fetch(b.d_run_length, B ? U + 1 : 1);
  if (what == "root") return fetch(b.d_root, U);
  if (what == "offset") return fetch(b.d_offset, U);
  if (what == "version") return fetch(t.d_version_, t.kStorageMax);
  if (what == "updates") return fetch(t.d_updates_, t.kNonLocalStorageMax);
  if (what == "shape" || what == "shape_exchanged") {
    py::array_t<long long> out(n);
    const size_t *src = what == "shape" ? b.h_shape : b.h_shape_exchanged;
    for (size_t i = 0; i < n; i++) out.mutable_data()[i] = (long long)src[i];
    return out;
  }
  if (what == "embedding" || what == "gradient") {
    const bool e = what == "embedding";
    const size_t cnt = (e ? t.kStorageMax : t.kNonLocalStorageMax) * t.kEmbeddingWidth;
    py::array_t<float> out(cnt);
    if (cnt) cudaMemcpy(out.mutable_data(), e ? t.d_embedding_ : t.d_gradient_, cnt * sizeof(float), cudaMemcpyDeviceToHost);
    return out;
  }
  throw std::runtime_error("unknown array " + what);
}

std::unique_ptr<HetuTable> make(int rank, int nrank, int device_id, const std::string &ip, int port, size_t length,
                                size_t width, long long pull_bound, long long push_bound,
                                py::array_t<worker_t, py::array::c_style | py::array::forcecast> root,
                                py::array_t<index_t, py::array::c_style | py::array::forcecast> storage, int init_kind,
                                float a, float b, float lr, int verbose) {
  SArray<worker_t> r(root.mutable_data(), root.size());
  SArray<index_t> s(storage.mutable_data(), storage.size());
  const InitType kinds[] = {InitType::kZero, InitType::kNormal, InitType::kUniform, InitType::kTruncatedNormal};
  Initializer init(kinds[init_kind], a, b);
  return std::make_unique<HetuTable>(rank, nrank, device_id, ip, port, length, width, pull_bound, push_bound, r, s,
                                     init, lr, verbose);
}

}  // namespace

PYBIND11_MODULE(hetuCTR_ref, m) {
  m.doc() = "the reference HetuCTR table, built unmodified, with array dumps (test infrastructure)";
  py::class_<HetuTable, std::unique_ptr<HetuTable>>(m, "HetuTable")
      .def(py::init(&make), py::arg("rank"), py::arg("nrank"), py::arg("device_id"), py::arg("ip"), py::arg("port"),
           py::arg("length"), py::arg("width"), py::arg("pull_bound"), py::arg("push_bound"), py::arg("root_arr"),
           py::arg("storage_arr"), py::arg("init_kind"), py::arg("init_a"), py::arg("init_b"),
           py::arg("learning_rate"), py::arg("verbose"))
      .def("preprocess",
           [](HetuTable &t, unsigned long ptr, size_t n) {
             py::gil_scoped_release rel;
             t.preprocess(reinterpret_cast<index_t *>(ptr), n);
           })
      .def("push_pull",
           [](HetuTable &t, unsigned long grad, unsigned long dst) {
             py::gil_scoped_release rel;
             t.pushPull(reinterpret_cast<embed_t *>(grad), reinterpret_cast<embed_t *>(dst));
           })
      // numpy in / numpy out: the binding stages gradients and pulled rows itself, so a driver script needs
      // no other CUDA library in the process
      .def("push_pull_np",
           [](HetuTable &t, py::object grad, size_t n_cur) {
             cudaSetDevice(t.device_id_);
             const size_t W = t.kEmbeddingWidth;
             float *d_grad = nullptr, *d_dst = nullptr;
             if (!grad.is_none()) {
               auto g = grad.cast<py::array_t<float, py::array::c_style | py::array::forcecast>>();
               cudaMalloc(&d_grad, std::max<size_t>(g.size(), 1) * sizeof(float));
               cudaMemcpy(d_grad, g.data(), g.size() * sizeof(float), cudaMemcpyHostToDevice);
             }
             cudaMalloc(&d_dst, std::max<size_t>(n_cur * W, 1) * sizeof(float));
             {
               py::gil_scoped_release rel;
               t.pushPull(d_grad, d_dst);
             }
             py::array_t<float> out({n_cur, W});
             cudaMemcpy(out.mutable_data(), d_dst, n_cur * W * sizeof(float), cudaMemcpyDeviceToHost);
             cudaFree(d_grad);
             cudaFree(d_dst);
             return out;
           },
           py::arg("grad"), py::arg("n_cur"))
      // Timed loop for the benchmark's reference arm: `steps` x (preprocess + push_pull) over the given key
      // batches (cycled) with real gradients, after `warmup` untimed steps.  host_buffers = false: keys,
      // gradients and dst are resident on the device before the clock starts; true: keys are passed as a
      // host pointer and gradients / pulled rows are copied from / to pinned host memory every step.
      // Every reference call ends with a stream synchronisation, so wall time around the loop is device time.
      .def("bench_loop",
           [](HetuTable &t, std::vector<py::array_t<long long, py::array::c_style | py::array::forcecast>> batches,
              py::array_t<float, py::array::c_style | py::array::forcecast> grad, int steps, int warmup,
              bool host_buffers) {
             cudaSetDevice(t.device_id_);
             const size_t W = t.kEmbeddingWidth, nb = batches.size();
             const size_t B = batches[0].size();
             std::vector<index_t *> dkeys(nb), hkeys(nb);
             for (size_t i = 0; i < nb; i++) {
               cudaMalloc(&dkeys[i], B * sizeof(index_t));
               cudaMemcpy(dkeys[i], batches[i].data(), B * sizeof(index_t), cudaMemcpyHostToDevice);
               cudaMallocHost(&hkeys[i], B * sizeof(index_t));
               memcpy(hkeys[i], batches[i].data(), B * sizeof(index_t));
             }
             float *dgrad[2], *ddst, *hgrad = nullptr, *hdst = nullptr;
             for (int i = 0; i < 2; i++) {
               cudaMalloc(&dgrad[i], B * W * sizeof(float));
               cudaMemcpy(dgrad[i], grad.data(), B * W * sizeof(float), cudaMemcpyHostToDevice);
             }
             cudaMalloc(&ddst, B * W * sizeof(float));
             if (host_buffers) {
               cudaMallocHost(&hgrad, B * W * sizeof(float));
               cudaMallocHost(&hdst, B * W * sizeof(float));
               memcpy(hgrad, grad.data(), B * W * sizeof(float));
             }
             double ms = 0;
             {
               py::gil_scoped_release rel;
               t.preprocess(dkeys[nb - 1], B);
               t.pushPull(nullptr, ddst);
               auto one = [&](int i) {
                 const size_t j = (size_t)i % nb;
                 if (host_buffers) {
                   t.preprocess(hkeys[j], B);
                   cudaMemcpy(dgrad[i & 1], hgrad, B * W * sizeof(float), cudaMemcpyHostToDevice);
                   t.pushPull(dgrad[i & 1], ddst);
                   cudaMemcpy(hdst, ddst, B * W * sizeof(float), cudaMemcpyDeviceToHost);
                 } else {
                   t.preprocess(dkeys[j], B);
                   t.pushPull(dgrad[i & 1], ddst);
                 }
               };
               for (int i = 0; i < warmup; i++) one(i);
               cudaDeviceSynchronize();
               auto t0 = std::chrono::steady_clock::now();
               for (int i = 0; i < steps; i++) one(i);
               cudaDeviceSynchronize();
               ms = std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - t0).count();
             }
             for (size_t i = 0; i < nb; i++) {
               cudaFree(dkeys[i]);
               cudaFreeHost(hkeys[i]);
             }
             cudaFree(dgrad[0]);
             cudaFree(dgrad[1]);
             cudaFree(ddst);
             if (hgrad) cudaFreeHost(hgrad);
             if (hdst) cudaFreeHost(hdst);
             return ms;
           },
           py::arg("batches"), py::arg("grad"), py::arg("steps"), py::arg("warmup"), py::arg("host_buffers"))
      .def("set_embedding",
           [](HetuTable &t, py::array_t<float, py::array::c_style | py::array::forcecast> rows) {
             cudaSetDevice(t.device_id_);
             cudaMemcpy(t.d_embedding_, rows.data(), rows.size() * sizeof(float), cudaMemcpyHostToDevice);
           })
      .def("dump", &dump, py::arg("what"), py::arg("prev") = false)
      .def("__repr__", &HetuTable::debugString);
  m.def("seed", [](unsigned long s) { __seed = s; });
}
