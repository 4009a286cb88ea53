// Python module `hetuCTR_partition`: same functions as the reference's (csrc/partition/pybind.cc:6-24) plus
// an optional seed and set_result().
#include <pybind11/numpy.h>
#include <pybind11/pybind11.h>

#include <memory>

#include "partition/partition.h"

namespace py = pybind11;
using hetuCTR::Partitioner;

namespace {

void check_contiguous(const py::array &a, const char *name) {
  if (!a.attr("flags").attr("c_contiguous").cast<bool>())
    throw std::runtime_error(std::string("Array not continuous in C: ") + name);
}

std::unique_ptr<Partitioner> make(py::array_t<int> data, py::array_t<float> comm, int n_part, int batch_size,
                                  unsigned long long seed) {
  check_contiguous(data, "_input_data");
  check_contiguous(comm, "_comm_mat");
  if (data.ndim() != 2) throw std::runtime_error("partition: data must be [n_data, n_slot]");
  if (comm.ndim() != 2 || comm.shape(0) != n_part || comm.shape(1) != n_part)
    throw std::runtime_error("partition: comm_mat must be [n_part, n_part]");
  return std::make_unique<Partitioner>(data.data(), (int)data.shape(0), (int)data.shape(1), comm.data(), n_part,
                                       batch_size, seed);
}

template <class T>
py::array_t<T> to_array(const std::vector<T> &v, std::vector<py::ssize_t> shape) {
  py::array_t<T> out(shape);
  std::copy(v.begin(), v.end(), out.mutable_data());
  return out;
}

}  // namespace

PYBIND11_MODULE(hetuCTR_partition, m) {
  m.doc() = "hetuCTR graph partition, deterministic implementation";
  py::class_<Partitioner>(m, "_PartitionStruct", py::module_local())
      .def("refine_data", [](Partitioner &p) { py::gil_scoped_release r; p.refineData(); })
      .def("refine_embed", [](Partitioner &p) { py::gil_scoped_release r; p.refineEmbed(); })
      .def("get_communication",
           [](Partitioner &p) { return to_array(p.communication(), {p.nPart(), p.nPart()}); })
      .def("get_priority", [](Partitioner &p) { return to_array(p.priority(), {p.nPart(), p.nEmbed()}); })
      .def("get_result",
           [](Partitioner &p) {
             return py::make_tuple(to_array(p.res_data_, {p.nData()}), to_array(p.res_embed_, {p.nEmbed()}));
           })
      .def("get_data_cnt", [](Partitioner &p) { return to_array(p.cnt_data_, {p.nPart()}); })
      .def("get_embed_cnt", [](Partitioner &p) { return to_array(p.cnt_embed_, {p.nPart()}); })
      .def("set_result", [](Partitioner &p, py::array_t<int, py::array::c_style | py::array::forcecast> d,
                            py::array_t<int, py::array::c_style | py::array::forcecast> e) {
        if (d.size() != p.nData() || e.size() != p.nEmbed()) throw std::runtime_error("set_result: wrong sizes");
        p.setResult(d.data(), e.data());
      });
  m.def("partition", &make, py::arg("data"), py::arg("comm_mat"), py::arg("n_part"), py::arg("batch_size"),
        py::arg("seed") = 0ull);
}
