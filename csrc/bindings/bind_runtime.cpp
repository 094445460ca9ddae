// Python view of the executor (`kern_b200._native.Runtime`).
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include "../manifest/verify.hpp"
#include "../runtime/runtime.hpp"

namespace py = pybind11;
using namespace kern;

static py::list copies_to_py(const std::vector<RowsCopy>& cs) {
  py::list out;
  for (auto& c : cs) out.append(py::make_tuple(c.src, c.dst, c.width, c.src_pitch, c.dst_pitch, c.rows));
  return out;
}

void bind_runtime(py::module_& m) {
  // push shapes (push.hpp): tuples (src, dst, width, src_pitch, dst_pitch, rows), byte offsets
  m.def("dealt_copies", [](const std::vector<std::tuple<int64_t, int64_t, int64_t, int64_t>>& runs, uint64_t row) {
    std::vector<pool::RowRun> rr;
    for (auto& r : runs) rr.push_back({std::get<0>(r), std::get<1>(r), std::get<2>(r), std::get<3>(r)});
    return copies_to_py(dealt_copies(rr, row));
  }, "runs (src_row, src_stride, dst_row, rows) of a deal as strided copies of `row`-byte rows, pieces of at most 64 KiB");
  m.def("split_copies", [](const std::vector<std::pair<uint64_t, uint64_t>>& segments, uint64_t of, uint64_t lines, uint64_t part) {
    return copies_to_py(Split(segments, of).copies(lines, part));
  }, "member `part`'s share of a slot of `lines` lines whose rows are sharded by heads over `of` members");
  m.def("split_line", [](const std::vector<std::pair<uint64_t, uint64_t>>& segments, uint64_t of) { return Split(segments, of).line(); });
  py::class_<Runtime, std::shared_ptr<Runtime>>(m, "Runtime")
      .def(py::init([](const std::string& manifest_text, const std::string& kernels_dir, int gpu,
                       std::map<std::string, std::pair<uint64_t, uint64_t>> topology, uint64_t tokens, uint64_t slots,
                       double memory_fraction, uint64_t stream, bool guard_bands) {
             Errors errs;
             Manifest mf = parse_manifest_text(manifest_text, errs);
             if (errs.empty()) errs = verify_manifest(mf);
             if (!errs.empty()) {
               std::string msg = "manifest does not verify:";
               for (auto& e : errs) msg += "\n  - " + e;
               throw py::value_error(msg);
             }
             std::map<std::string, GroupRank> topo;
             for (auto& kv : topology) topo[kv.first] = GroupRank{kv.second.first, kv.second.second};
             Capacity cap;
             cap.tokens = tokens;
             cap.slots = slots;
             cap.memory_fraction = memory_fraction;
             cap.guard_bands = guard_bands;
             return std::make_shared<Runtime>(std::move(mf), kernels_dir, gpu, std::move(topo), cap, stream);
           }),
           py::arg("manifest"), py::arg("kernels"), py::arg("gpu") = 0,
           py::arg("topology") = std::map<std::string, std::pair<uint64_t, uint64_t>>(), py::arg("tokens") = 0,
           py::arg("slots") = 0, py::arg("memory_fraction") = 0.9, py::arg("stream") = 0, py::arg("guard_bands") = false)
      .def("manifest_json", [](Runtime& r) { return manifest_to_json(r.manifest()).dump(1); })
      .def("protocol_json", [](Runtime& r) -> py::object {
        if (!r.protocol()) return py::none();
        return py::str(r.protocol()->to_json().dump());
      })
      .def_property_readonly("stream", &Runtime::stream)
      .def_property_readonly("page_unit", &Runtime::page_unit)
      .def_property_readonly("pages", &Runtime::pages)
      .def_property_readonly("slots", &Runtime::slots)
      .def_property_readonly("launches_total", &Runtime::launches_total)
      .def_property_readonly("graphs", &Runtime::graphs)
      .def_property_readonly("awaits_host", &Runtime::awaits_host)
      .def_property_readonly("weights_loaded", &Runtime::weights_loaded)
      .def_property_readonly("peers_connected", &Runtime::peers_connected)
      .def("rank", &Runtime::rank)
      .def("banner", &Runtime::banner)
      .def("load_weights", [](Runtime& r, std::vector<std::string> paths) {
        py::gil_scoped_release rel;
        r.load_weights(paths);
      })
      .def("region", &Runtime::region)
      .def("write_input", [](Runtime& r, const std::string& name, py::buffer data, size_t offset) {
        py::buffer_info info = data.request();
        r.write_input(name, info.ptr, (size_t)info.size * (size_t)info.itemsize, offset);
      }, py::arg("name"), py::arg("data"), py::arg("offset") = 0)
      // raw pointer form: pinned host memory owned by the caller (a torch pinned tensor)
      .def("write_input_ptr", [](Runtime& r, const std::string& name, uint64_t host_ptr, size_t bytes, size_t offset) {
        r.write_input(name, reinterpret_cast<const void*>(host_ptr), bytes, offset);
      }, py::arg("name"), py::arg("host_ptr"), py::arg("bytes"), py::arg("offset") = 0)
      .def("read_output", [](Runtime& r, const std::string& name, size_t bytes, size_t offset) {
        std::string out(bytes, '\0');
        {
          py::gil_scoped_release rel;
          r.read_output(name, &out[0], bytes, offset);
        }
        return py::bytes(out);
      }, py::arg("name"), py::arg("bytes"), py::arg("offset") = 0)
      .def("read_output_ptr", [](Runtime& r, const std::string& name, uint64_t host_ptr, size_t bytes, size_t offset) {
        py::gil_scoped_release rel;
        r.read_output(name, reinterpret_cast<void*>(host_ptr), bytes, offset);
      }, py::arg("name"), py::arg("host_ptr"), py::arg("bytes"), py::arg("offset") = 0)
      .def("synchronize", [](Runtime& r) {
        py::gil_scoped_release rel;
        r.synchronize();
      })
      .def("run_once_programs", &Runtime::run_once_programs)
      .def("issue_range", [](Runtime& r, const std::string& program, const VarMap& vars, size_t lo, size_t hi) {
        return r.issue_range(program, vars, lo, hi);
      })
      .def("issue", [](Runtime& r, const std::string& program, const VarMap& vars, bool eager) {
        return r.issue(program, vars, eager);
      }, py::arg("program"), py::arg("vars"), py::arg("eager") = false)
      .def("run", [](Runtime& r, const std::string& program, const VarMap& vars) {
        size_t n = r.issue(program, vars, false);
        py::gil_scoped_release rel;
        r.synchronize();
        return n;
      })
      .def("issue_timed", [](Runtime& r, const std::string& program, const VarMap& vars) {
        std::vector<std::tuple<std::string, std::string, float, size_t>> out;
        for (auto& c : r.issue_timed(program, vars)) out.emplace_back(c.label, c.op, c.ms, c.launches);
        return out;
      })
      .def("is_captured", &Runtime::is_captured)
      .def("enqueue_after", &Runtime::enqueue_after)
      .def("zero_slot", &Runtime::zero_slot)
      .def("copy_pages", &Runtime::copy_pages)
      .def("copy_slot", &Runtime::copy_slot)
      .def("export_handles", [](Runtime& r) {
        py::dict d;
        for (auto& kv : r.export_handles()) d[py::str(kv.first)] = py::bytes(kv.second);
        return d;
      })
      .def("connect", [](Runtime& r, const std::string& group, std::vector<std::map<std::string, py::bytes>> members) {
        std::vector<std::map<std::string, std::string>> ms;
        for (auto& mm : members) {
          std::map<std::string, std::string> one;
          for (auto& kv : mm) one[kv.first] = std::string(kv.second);
          ms.push_back(std::move(one));
        }
        r.connect(group, ms);
      })
      .def("check_guards", &Runtime::check_guards)
      .def("checked_failures", &Runtime::checked_failures)
      .def_property_readonly("checked", &Runtime::checked)
      .def("export_region", [](Runtime& r, const std::string& name) { return py::bytes(r.export_region(name)); })
      .def("import_region", [](Runtime& r, py::bytes h) { return r.import_region(std::string(h)); })
      .def("push_unit", &Runtime::push_unit)
      .def("push_bytes", &Runtime::push_bytes)
      .def("push_copies", [](Runtime& r, const std::string& state, uint64_t src_off, uint64_t dst_base, uint64_t dst_bytes,
                             const std::vector<std::tuple<uint64_t, uint64_t, uint64_t, uint64_t, uint64_t, uint64_t>>& copies) {
        std::vector<RowsCopy> cs;
        for (auto& c : copies) cs.push_back({std::get<0>(c), std::get<1>(c), std::get<2>(c), std::get<3>(c), std::get<4>(c), std::get<5>(c)});
        r.push_copies(state, src_off, dst_base, dst_bytes, cs);
      })
      .def("bind_host", &Runtime::bind_host);
}
