// Python view of the pool library: Pool / Lease / Checkpoint / Prefix / deal.
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include "../pool/deal.hpp"
#include "../pool/prefix.hpp"

namespace py = pybind11;
using namespace kern::pool;

namespace {

py::dict copies_dict(const Copies& c) {
  py::dict d;
  d["pages"] = c.pages;
  d["half_tokens"] = c.half_tokens;
  d["slot"] = c.slot ? py::cast(*c.slot) : py::none();
  return d;
}

struct PyLease {
  Lease l;
};

}  // namespace

void bind_pool(py::module_& m) {
  py::class_<Checkpoint>(m, "Checkpoint")
      .def_readonly("len", &Checkpoint::len)
      .def_readonly("pages", &Checkpoint::pages)
      .def_property_readonly("has_slot", &Checkpoint::has_slot)
      .def_property_readonly("slot", &Checkpoint::slot_id)
      .def("page_ids", &Checkpoint::page_ids)
      .def("usable_at", &Checkpoint::usable_at);

  py::class_<PyLease, std::shared_ptr<PyLease>>(m, "Lease")
      .def_property_readonly("live", [](PyLease& p) { return p.l.live(); })
      .def_property_readonly("pages", [](PyLease& p) { return p.l.pages(); })
      .def_property_readonly("shared_pages", [](PyLease& p) { return p.l.shared_pages(); })
      .def_property_readonly("capacity", [](PyLease& p) { return p.l.capacity(); })
      .def_property_readonly("prefix", [](PyLease& p) { return p.l.prefix(); })
      .def_property_readonly("slot", [](PyLease& p) { return p.l.slot(); })
      .def("slot_of", [](PyLease& p, uint64_t pos) { return p.l.slot_of(pos); })
      .def("slots_of", [](PyLease& p, uint64_t lo, uint64_t hi) {
        std::vector<int64_t> out;
        out.reserve(hi > lo ? hi - lo : 0);
        for (uint64_t i = lo; i < hi; ++i) out.push_back(p.l.slot_of(i));
        return out;
      })
      .def("release", [](PyLease& p) { p.l.release(); });

  static py::exception<Denied> denied(m, "Denied", PyExc_RuntimeError);
  py::register_exception_translator([](std::exception_ptr p) {
    try {
      if (p) std::rethrow_exception(p);
    } catch (const Denied& e) {
      static const char* names[] = {"busy", "exceeds_row", "exceeds_pool"};
      PyObject* args = Py_BuildValue("(ss)", e.what(), names[e.why]);
      PyErr_SetObject(denied.ptr(), args);
      Py_XDECREF(args);
    }
  });

  py::class_<Pool, std::shared_ptr<Pool>>(m, "Pool")
      .def(py::init<uint64_t, uint64_t, uint64_t, uint64_t>(), py::arg("unit"), py::arg("pages"), py::arg("slots") = 0,
           py::arg("row_pages") = 0)
      .def_property_readonly("unit", &Pool::unit)
      .def_property_readonly("total_pages", &Pool::total_pages)
      .def_property_readonly("free_pages", &Pool::free_pages)
      .def_property_readonly("total_slots", &Pool::total_slots)
      .def_property_readonly("free_slots", &Pool::free_slots)
      .def_property_readonly("stateful", &Pool::stateful)
      .def("pages_for", &Pool::pages_for)
      .def("room", &Pool::room, py::arg("pages"), py::arg("slot") = true)
      .def("lease", [](Pool& p, uint64_t tokens) {
        auto out = std::make_shared<PyLease>();
        out->l = p.lease(tokens);
        return out;
      })
      .def("extend", [](Pool& p, PyLease& l, uint64_t tokens) { p.extend(l.l, tokens); })
      .def("checkpoint", [](Pool& p, PyLease& l, uint64_t len) {
        auto r = p.checkpoint(l.l, len);
        return py::make_tuple(r.first, copies_dict(r.second));
      })
      .def("retire", [](Pool& p, PyLease& l, uint64_t len) { return p.retire(std::move(l.l), len); })
      .def("restore", [](Pool& p, const Checkpoint& c, uint64_t len, uint64_t tokens) {
        auto r = p.restore(c, len, tokens);
        auto out = std::make_shared<PyLease>();
        out->l = std::move(r.first);
        return py::make_tuple(out, copies_dict(r.second));
      })
      .def("fork", [](Pool& p, PyLease& parent, uint64_t len, uint64_t tokens) {
        auto r = p.fork(parent.l, len, tokens);
        auto out = std::make_shared<PyLease>();
        out->l = std::move(r.first);
        return py::make_tuple(out, copies_dict(r.second));
      });

  using PyPrefix = Prefix<py::object>;
  py::class_<PyPrefix>(m, "Prefix")
      .def(py::init<uint64_t>(), py::arg("unit"))
      .def_property_readonly("unit", &PyPrefix::unit)
      .def("__len__", &PyPrefix::size)
      .def("insert", &PyPrefix::insert, py::arg("key"), py::arg("kept"), py::arg("has_slot"), py::arg("len"))
      .def("lookup", [](PyPrefix& p, const Tokens& prompt, uint64_t at_most) -> py::object {
        auto h = p.lookup(prompt, at_most);
        if (!h) return py::none();
        return py::make_tuple(h->len, h->found);
      }, py::arg("prompt"), py::arg("at_most") = UINT64_MAX)
      .def("evict", &PyPrefix::evict)
      .def("remove", &PyPrefix::remove)
      .def("clear", &PyPrefix::clear);

  py::class_<Interleave>(m, "Interleave")
      .def(py::init<uint64_t>())
      .def_readonly("w", &Interleave::w)
      .def("owner", &Interleave::owner)
      .def("local", &Interleave::local)
      .def("len", &Interleave::len);
  m.def("deal", [](const std::vector<int32_t>& src_ids, uint64_t src_unit, const std::vector<int32_t>& dst_ids,
                   uint64_t dst_unit, uint64_t w, uint64_t member, uint64_t len) {
    auto runs = deal(PagesView{src_ids, src_unit}, PagesView{dst_ids, dst_unit}, Interleave(w), member, len);
    std::vector<std::tuple<int64_t, int64_t, int64_t, int64_t>> out;
    for (auto& r : runs) out.emplace_back(r.src_row, r.src_stride, r.dst_row, r.rows);
    return out;
  });
}
