// Python bindings of the native runtime: `_exo_native` (bus, pidfile, NVML topology).
// Same five bus calls as the reference's PyO3 NetworkingHandle (rust/exo_rs/exo_rs.pyi:35-56:
// new / recv / subscribe / unsubscribe / publish); recv is exposed as an event fd the asyncio loop
// can watch plus a non-blocking pop, so no thread ever blocks holding the GIL.
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include "bus.h"

namespace py = pybind11;
using namespace exo;

PYBIND11_MODULE(_exo_native, m) {
  m.doc() = "exo-b200 native runtime: message bus, pidfile, NVML topology";
  m.def("namespace_hash", &namespace_hash);
  m.def("valid_identity", &valid_identity);

  py::class_<Bus>(m, "Bus")
      .def(py::init<const std::string&, const std::string&, int, int>(), py::arg("identity"), py::arg("namespace"),
           py::arg("listen_port") = 0, py::arg("discovery_port") = 0)
      .def_property_readonly("listen_port", &Bus::listen_port)
      .def_property_readonly("event_fd", &Bus::event_fd)
      .def("try_recv",
           [](Bus& b) -> py::object {
             BusEvent e;
             if (!b.try_recv(&e)) return py::none();
             if (e.kind == BusEvent::Connection) return py::make_tuple("connection", e.peer, e.connected);
             if (e.kind == BusEvent::Discovered) return py::make_tuple("discovered", e.peer, e.data);
             return py::make_tuple("message", e.topic, py::bytes(e.data));
           })
      .def("connect", [](Bus& b, const std::string& host, int port) {
             py::gil_scoped_release r;
             return b.connect_to(host, port);
           })
      .def("subscribe", [](Bus& b, const std::string& t) { py::gil_scoped_release r; b.subscribe(t); })
      .def("unsubscribe", [](Bus& b, const std::string& t) { py::gil_scoped_release r; b.unsubscribe(t); })
      .def("publish", [](Bus& b, const std::string& t, const py::bytes& d) {
             std::string data = d;
             py::gil_scoped_release r;
             return b.publish(t, data);
           })
      .def("peers", &Bus::peers)
      .def("close", [](Bus& b) { py::gil_scoped_release r; b.close(); });

  py::register_exception<std::runtime_error>(m, "NativeError");
  py::class_<Pidfile>(m, "Pidfile")
      .def(py::init<const std::string&>())
      .def("write", &Pidfile::write)
      .def("as_raw_fd", &Pidfile::raw_fd)
      .def("close", &Pidfile::close);

  py::class_<GpuInfo>(m, "GpuInfo")
      .def_readonly("index", &GpuInfo::index)
      .def_readonly("name", &GpuInfo::name)
      .def_readonly("uuid", &GpuInfo::uuid)
      .def_readonly("mem_total", &GpuInfo::mem_total)
      .def_readonly("mem_free", &GpuInfo::mem_free)
      .def_readonly("power_mw", &GpuInfo::power_mw)
      .def_readonly("temp_c", &GpuInfo::temp_c)
      .def_readonly("util_pct", &GpuInfo::util_pct)
      .def_readonly("sm_mhz", &GpuInfo::sm_mhz)
      .def_readonly("nvlink_peers_links", &GpuInfo::nvlink_peers_links)
      .def_readonly("p2p_ok", &GpuInfo::p2p_ok)
      .def_readonly("active_links", &GpuInfo::active_links);
  m.def("nvml_enumerate", []() {
    std::string err;
    auto v = nvml_enumerate(&err);
    return py::make_tuple(v, err);
  });
}
