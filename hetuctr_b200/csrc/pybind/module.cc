// Python module `hetuCTR`: same classes, constructor keywords and methods as the reference's module
// (csrc/pybind/pybind.cu:42-79, csrc/pybind/container.h:10-37), bound to the new HetuTable.
#include <pybind11/numpy.h>
#include <pybind11/pybind11.h>

#include <future>
#include <memory>

#include "core/hetu_table.h"
#include "utils/thread_pool.h"

namespace py = pybind11;
using namespace hetuCTR;

namespace {

// The table plus the one-thread queue behind async_* (csrc/pybind/container.h:24-37).
class TableContainer : public HetuTable {
 public:
  using HetuTable::HetuTable;

  void pushPull(unsigned long grad, unsigned long dst) {
    py::gil_scoped_release release;
    HetuTable::pushPull(reinterpret_cast<embed_t *>(grad), reinterpret_cast<embed_t *>(dst));
  }
  void preprocess(unsigned long data_ptr, size_t batch_size) {
    py::gil_scoped_release release;
    HetuTable::preprocess(reinterpret_cast<index_t *>(data_ptr), batch_size);
  }
  std::future<void> pushPullAsync(unsigned long grad, unsigned long dst) {
    if (!pool_) pool_ = std::make_unique<ThreadPool>(1);
    return pool_->Enqueue([this, grad, dst] {
      HetuTable::pushPull(reinterpret_cast<embed_t *>(grad), reinterpret_cast<embed_t *>(dst));
    });
  }
  std::future<void> preprocessAsync(unsigned long data_ptr, size_t batch_size) {
    if (!pool_) pool_ = std::make_unique<ThreadPool>(1);
    return pool_->Enqueue(
        [this, data_ptr, batch_size] { HetuTable::preprocess(reinterpret_cast<index_t *>(data_ptr), batch_size); });
  }
  ~TableContainer() { pool_.reset(); }

 private:
  std::unique_ptr<ThreadPool> pool_;
};

void check_contiguous(const py::array &a, const char *name) {
  if (!a.attr("flags").attr("c_contiguous").cast<bool>())
    throw std::runtime_error(std::string("Array not continuous in C: ") + name);
}

std::unique_ptr<TableContainer> makeTable(const int rank, const int nrank, const int device_id, const std::string &ip,
                                          const int port, const size_t embedding_length,
                                          const size_t embedding_width, const version_t pull_bound,
                                          const version_t push_bound, py::array_t<worker_t> root_id_arr,
                                          py::array_t<index_t> storage_id_arr, const Initializer &init,
                                          const embed_t learning_rate, const int verbose) {
  check_contiguous(root_id_arr, "root_id_arr");
  check_contiguous(storage_id_arr, "storage_id_arr");
  return std::make_unique<TableContainer>(rank, nrank, device_id, ip, port, embedding_length, embedding_width,
                                          pull_bound, push_bound, root_id_arr.data(), (size_t)root_id_arr.size(),
                                          storage_id_arr.data(), (size_t)storage_id_arr.size(), init, learning_rate,
                                          verbose);
}

}  // namespace

PYBIND11_MODULE(hetuCTR, m) {
  m.doc() = "hetuCTR embedding table, B200-native implementation";

  typedef std::future<void> wait_t;
  py::class_<wait_t>(m, "_waittype").def("wait", [](wait_t &w) {
    py::gil_scoped_release release;
    w.get();  // rethrows a failure of the queued call
  });

  py::enum_<InitType>(m, "InitType", py::module_local())
      .value("Zero", InitType::kZero)
      .value("Normal", InitType::kNormal)
      .value("TruncatedNormal", InitType::kTruncatedNormal)
      .value("Uniform", InitType::kUniform);

  py::class_<Initializer, std::unique_ptr<Initializer>>(m, "Initializer", py::module_local())
      .def(py::init([](InitType t, float a, float b) { return std::make_unique<Initializer>(t, a, b); }));

  py::class_<TableContainer, std::unique_ptr<TableContainer>>(m, "HetuTable", py::module_local())
      .def(py::init(&makeTable), py::arg("rank"), py::arg("nrank"), py::arg("device_id"), py::arg("ip"),
           py::arg("port"), py::arg("length"), py::arg("width"), py::arg("pull_bound"), py::arg("push_bound"),
           py::arg("root_arr"), py::arg("storage_arr"), py::arg("init"), py::arg("learning_rate"),
           py::arg("verbose"))
      .def("preprocess", &TableContainer::preprocess)
      .def("push_pull", &TableContainer::pushPull)
      .def("async_push_pull", &TableContainer::pushPullAsync)
      .def("async_preprocess", &TableContainer::preprocessAsync)
      .def("__repr__", &TableContainer::debugString)
      .def("debug", &TableContainer::debugStringFull)
      // extensions (not in the reference)
      .def("dump",
           [](TableContainer &t, const std::string &what, bool prev) -> py::array {
             const long long n = t.dump(what, prev, nullptr);
             if (what == "embedding" || what == "gradient") {
               py::array_t<float> out(n);
               t.dump(what, prev, out.mutable_data());
               return out;
             }
             py::array_t<long long> out(n);
             t.dump(what, prev, out.mutable_data());
             return out;
           },
           py::arg("what"), py::arg("prev") = false)
      .def("set_embedding", [](TableContainer &t, py::array_t<float, py::array::c_style | py::array::forcecast> rows) {
        if ((size_t)rows.size() != t.kStorageMax * t.kEmbeddingWidth)
          throw std::runtime_error("set_embedding: expected stored_rows * width values");
        t.setEmbedding(rows.data());
      })
      // checkpoint of this rank's learned state (the reference has none)
      .def("export_state", [](TableContainer &t, const std::string &path) { t.exportState(path); },
           py::arg("path"), py::call_guard<py::gil_scoped_release>())
      .def("import_state", [](TableContainer &t, const std::string &path) { t.importState(path); },
           py::arg("path"), py::call_guard<py::gil_scoped_release>());

  m.def("seed", [](unsigned long seed) { set_seed(seed); });
}
