// Python view of the device layer: a thin, typed launcher that the op wrappers, tests and the
// Python framework layer use to run the in-tree sm_100a cubins on PyTorch tensors (same primary
// context, same stream).
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include "../runtime/cupti_trace.hpp"
#include "../runtime/device.hpp"

namespace py = pybind11;
using namespace kern;

namespace {

struct PyModule {
  CUmodule m;
};
struct PyFunction {
  CUfunction f;
  std::string name;
};
struct PyGraph {
  std::shared_ptr<Device> dev;
  CUgraphExec g = nullptr;
  size_t nodes = 0;
  ~PyGraph() {
    if (g) dev->graph_destroy(g);
  }
};

}  // namespace

void bind_device(py::module_& m) {
  m.def("cuda_available", [] { return Cuda::available(); });
  // kernel activity tracing (CUPTI by dlopen): start / collect / stop; records are
  // (name, start_ns, end_ns, stream, (gx, gy, gz), (bx, by, bz), registers, shared_bytes)
  m.def("cupti_available", [] {
    std::string why;
    const bool ok = CuptiTrace::get().available(&why);
    return py::make_tuple(ok, why);
  });
  m.def("cupti_start", [] { CuptiTrace::get().start(); });
  auto to_py = [](const std::vector<KernelRecord>& recs) {
    py::list out;
    for (auto& r : recs)
      out.append(py::make_tuple(r.name, r.start_ns, r.end_ns, r.stream, py::make_tuple(r.grid[0], r.grid[1], r.grid[2]),
                                py::make_tuple(r.block[0], r.block[1], r.block[2]), r.registers, r.shared_bytes));
    return out;
  };
  m.def("cupti_collect", [to_py] {
    std::vector<KernelRecord> recs;
    {
      py::gil_scoped_release rel;
      recs = CuptiTrace::get().collect();
    }
    return to_py(recs);
  });
  m.def("cupti_stop", [to_py] {
    std::vector<KernelRecord> recs;
    {
      py::gil_scoped_release rel;
      recs = CuptiTrace::get().stop();
    }
    return to_py(recs);
  });
  m.def("cupti_dropped", [] { return CuptiTrace::get().dropped(); });

  py::class_<PyModule>(m, "Module");
  py::class_<PyFunction>(m, "Function").def_readonly("name", &PyFunction::name);
  py::class_<PyGraph, std::shared_ptr<PyGraph>>(m, "Graph").def_readonly("nodes", &PyGraph::nodes);

  py::class_<Device, std::shared_ptr<Device>>(m, "Device")
      .def(py::init<int>(), py::arg("gpu") = 0)
      .def_property_readonly("gpu", &Device::gpu)
      .def_property_readonly("sm_count", &Device::sm_count)
      .def_property_readonly("cc", &Device::cc)
      .def("make_current", &Device::make_current)
      .def("load_module", [](Device& d, py::bytes image) { return PyModule{d.load_module(image)}; })
      .def("function",
           [](Device& d, PyModule& mod, const std::string& entry) {
             return PyFunction{d.function(mod.m, entry), entry};
           })
      .def("entries", [](Device& d, PyModule& mod) { return d.entries(mod.m); })
      .def("param_sizes", [](Device& d, PyFunction& f) { return d.param_sizes(f.f); })
      .def(
          "launch",
          [](Device& d, PyFunction& f, std::array<unsigned, 3> grid, std::array<unsigned, 3> block,
             unsigned shared_mem, uint64_t stream, std::vector<py::bytes> params,
             std::array<unsigned, 3> cluster, bool pdl) {
            LaunchDims dims;
            for (int i = 0; i < 3; ++i) {
              dims.grid[i] = grid[i];
              dims.block[i] = block[i];
              dims.cluster[i] = cluster[i];
            }
            dims.shared_mem = shared_mem;
            dims.pdl = pdl;
            // every parameter image is copied into 64-byte aligned storage (tensor maps need it)
            std::vector<std::string> hold;
            hold.reserve(params.size());
            size_t total = 0;
            for (auto& p : params) {
              hold.emplace_back(p);
              total += (hold.back().size() + 63) / 64 * 64;
            }
            std::vector<uint8_t> arena(total + 64);
            uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(arena.data()) + 63) & ~uintptr_t(63));
            std::vector<void*> ptrs;
            size_t off = 0;
            for (auto& h : hold) {
              std::memcpy(base + off, h.data(), h.size());
              ptrs.push_back(base + off);
              off += (h.size() + 63) / 64 * 64;
            }
            d.launch(f.f, dims, reinterpret_cast<CUstream>(stream), ptrs.data());
          },
          py::arg("function"), py::arg("grid"), py::arg("block"), py::arg("shared_mem"),
          py::arg("stream"), py::arg("params"),
          py::arg("cluster") = std::array<unsigned, 3>{1, 1, 1}, py::arg("pdl") = false)
      .def(
          "encode_tensor_map",
          [](Device& d, uint64_t base, int dtype, std::vector<uint64_t> dims,
             std::vector<uint64_t> strides, std::vector<uint32_t> box, int swizzle, int l2_promotion,
             bool oob_nan) {
            TensorMapSpec s;
            s.dtype = dtype;
            s.dims = std::move(dims);
            s.strides = std::move(strides);
            s.box = std::move(box);
            s.swizzle = swizzle;
            s.l2_promotion = l2_promotion;
            s.oob_nan = oob_nan;
            auto a = d.encode_tensor_map(base, s);
            return py::bytes(reinterpret_cast<const char*>(a.data()), a.size());
          },
          py::arg("base"), py::arg("dtype"), py::arg("dims"), py::arg("strides"), py::arg("box"),
          py::arg("swizzle") = 0, py::arg("l2_promotion") = 0, py::arg("oob_nan") = false)
      .def("alloc", &Device::alloc)
      .def("free", &Device::free)
      .def("mem_info", &Device::mem_info)
      .def("ipc_export", [](Device& d, uint64_t p) { return py::bytes(d.ipc_export(p)); })
      .def("ipc_import", [](Device& d, py::bytes h) { return d.ipc_import(h, nullptr); })
      .def("ipc_close", &Device::ipc_close)
      .def("stream_create", [](Device& d) { return (uint64_t)d.stream_create(); })
      .def("stream_sync", [](Device& d, uint64_t s) {
        py::gil_scoped_release rel;
        d.stream_sync((CUstream)s);
      })
      .def("begin_capture", [](Device& d, uint64_t s) { d.begin_capture((CUstream)s); })
      .def("end_capture",
           [](std::shared_ptr<Device> d, uint64_t s) {
             auto g = std::make_shared<PyGraph>();
             g->dev = d;
             g->g = d->end_capture((CUstream)s, &g->nodes);
             return g;
           })
      .def("graph_launch", [](Device& d, PyGraph& g, uint64_t s) { d.graph_launch(g.g, (CUstream)s); });
}
