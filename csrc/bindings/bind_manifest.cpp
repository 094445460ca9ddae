// Python view of the manifest library: parse + verify (every diagnostic at once), the protocol
// projection as a plain dict-shaped JSON document, re-serialisation, `cut`, candidates.
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include <chrono>

#include "../manifest/cut.hpp"
#include "../manifest/protocol.hpp"
#include "../manifest/values.hpp"
#include "../manifest/verify.hpp"

namespace py = pybind11;
using namespace kern;

namespace {

struct PyManifest {
  std::shared_ptr<Manifest> m;
  std::string to_json(int indent) const { return manifest_to_json(*m).dump(indent); }
};

}  // namespace

void bind_manifest(py::module_& m) {
  m.attr("SCHEMA_VERSION") = SCHEMA_VERSION;

  py::class_<PyManifest>(m, "Manifest")
      .def("to_json", &PyManifest::to_json, py::arg("indent") = 1)
      .def_property_readonly("model", [](const PyManifest& p) { return p.m->model; })
      .def("protocol",
           [](const PyManifest& p, bool sampled) {
             Errors errs;
             auto pr = protocol_check(*p.m, sampled, errs);
             if (!pr) {
               std::string msg = "manifest does not fit the serving protocol:";
               for (auto& e : errs) msg += "\n  - " + e;
               throw py::value_error(msg);
             }
             return pr->to_json().dump();
           },
           py::arg("sampled") = true)
      .def("self_hosted",
           [](const PyManifest& p) { return PyManifest{std::make_shared<Manifest>(self_hosted(*p.m, 0))}; })
      .def("cut",
           [](const PyManifest& p, std::vector<size_t> at) {
             Errors errs;
             auto stages = cut_manifest(*p.m, at, errs);
             if (!errs.empty()) {
               std::string msg = "cannot cut:";
               for (auto& e : errs) msg += "\n  - " + e;
               throw py::value_error(msg);
             }
             std::vector<PyManifest> out;
             for (auto& s : stages) out.push_back(PyManifest{std::make_shared<Manifest>(std::move(s))});
             return out;
           })
      .def("splice",
           [](const PyManifest& p, const std::string& candidate_json) {
             Errors errs;
             Manifest out = splice_candidate(*p.m, candidate_json, errs);
             if (!errs.empty()) {
               std::string msg = "cannot splice candidate:";
               for (auto& e : errs) msg += "\n  - " + e;
               throw py::value_error(msg);
             }
             return PyManifest{std::make_shared<Manifest>(std::move(out))};
           });

  // -> (manifest | None, [diagnostics])
  m.def("verify", [](const std::string& text, bool strict_multicast) -> py::object {
    Errors errs;
    auto mf = std::make_shared<Manifest>();
    {
      py::gil_scoped_release rel;
      *mf = parse_manifest_text(text, errs);
      if (errs.empty()) errs = verify_manifest(*mf, strict_multicast);
    }
    if (errs.empty()) return py::make_tuple(py::cast(PyManifest{mf}), errs);
    return py::make_tuple(py::none(), errs);
  }, py::arg("text"), py::arg("strict_multicast") = false);

  // parse only (typed, constants expanded); diagnostics of the parse stage
  m.def("parse", [](const std::string& text) -> py::object {
    Errors errs;
    auto mf = std::make_shared<Manifest>(parse_manifest_text(text, errs));
    return py::make_tuple(py::cast(PyManifest{mf}), errs);
  });

  // seconds for `repeats` parse+verify passes over the text (the "millisecond verify" figure)
  m.def("verify_seconds", [](const std::string& text, int repeats) {
    auto t0 = std::chrono::steady_clock::now();
    size_t n = 0;
    for (int i = 0; i < repeats; ++i) {
      Errors errs;
      Manifest mf = parse_manifest_text(text, errs);
      if (errs.empty()) errs = verify_manifest(mf);
      n += errs.size();
    }
    auto t1 = std::chrono::steady_clock::now();
    (void)n;
    return std::chrono::duration<double>(t1 - t0).count() / std::max(1, repeats);
  });

  m.def("registry_url", [](const std::string& source) -> py::object {
    std::string url, err;
    int r = registry_ref_parse(source, url, err);
    if (r < 0) throw py::value_error(err);
    if (r == 0) return py::none();
    return py::str(url);
  });

  // dtype codecs used by comparisons
  m.def("ulp_distance", [](const std::string& dtype, py::bytes a, py::bytes b) {
    DType dt;
    if (!dtype_parse(dtype, dt)) throw py::value_error("unknown dtype");
    std::string sa = a, sb = b;
    return values::max_ulp_distance(dt, sa, sb);
  });
  m.def("decode_values", [](const std::string& dtype, py::bytes a) {
    DType dt;
    if (!dtype_parse(dtype, dt)) throw py::value_error("unknown dtype");
    std::string sa = a;
    return values::decode(dt, sa);
  });
  m.def("encode_values", [](const std::string& dtype, std::vector<double> v) {
    DType dt;
    if (!dtype_parse(dtype, dt)) throw py::value_error("unknown dtype");
    return py::bytes(values::encode(dt, v));
  });
}
