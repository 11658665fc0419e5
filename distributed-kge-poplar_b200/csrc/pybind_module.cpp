// Python module `libpoplar_kge` over the C ABI: the class and method names, argument names
// and exception types of the reference's binding (src/lib.cpp:38-52), so that its Python
// wrapper and scripts run unchanged on top of this engine.
#include <pybind11/numpy.h>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include <list>
#include <string>
#include <vector>

#include "kge_b200.h"

namespace py = pybind11;

namespace {

[[noreturn]] void raise(int status, const char* message) {
    // std::invalid_argument surfaces as ValueError in the reference, everything else as RuntimeError.
    if (status == KGE_INVALID_ARGUMENT) throw py::value_error(message);
    throw std::runtime_error(message);
}

class Engine {
   public:
    Engine(const py::dict& settings, const std::string& gp_folder) {
        std::list<std::string> keep;  // owns the strings the kge_setting entries point at
        std::vector<kge_setting> flat;
        auto add = [&](const std::string& key, py::handle value) {
            keep.push_back(key);
            kge_setting s{keep.back().c_str(), KGE_SET_STRING, nullptr, 0.0, 0ull};
            if (py::isinstance<py::bool_>(value) || py::isinstance(value, py::module_::import("numpy").attr("bool_"))) {
                s.type = KGE_SET_BOOL;
                s.u = value.cast<bool>() ? 1 : 0;
            } else if (py::isinstance<py::str>(value)) {
                keep.push_back(value.cast<std::string>());
                s.s = keep.back().c_str();
            } else if (py::isinstance<py::float_>(value) || py::isinstance(value, py::module_::import("numpy").attr("floating"))) {
                s.type = KGE_SET_FLOAT;
                s.f = value.cast<double>();
            } else if (PyIndex_Check(value.ptr())) {
                const long long v = value.cast<long long>();
                if (v < 0) throw py::value_error("Key '" + key + "' holds a negative integer");
                s.type = KGE_SET_UNSIGNED;
                s.u = (unsigned long long)v;
            } else {
                throw py::value_error("Key '" + key + "' holds value of unexpected type.");
            }
            flat.push_back(s);
        };
        for (auto item : settings) {
            const std::string key = py::str(item.first);
            if (py::isinstance<py::dict>(item.second)) {
                // the one map-valued setting, training.learning_rate_modifiers: {name: float}
                for (auto entry : item.second.cast<py::dict>()) {
                    const std::string sub = key + "." + std::string(py::str(entry.first));
                    add(sub, py::float_(entry.second.cast<double>()));
                }
            } else {
                add(key, item.second);
            }
        }
        const int status = kge_create(flat.data(), flat.size(), gp_folder.c_str(), &engine_);
        if (status != KGE_OK) raise(status, kge_last_error(nullptr));
    }
    ~Engine() { kge_destroy(engine_); }
    Engine(const Engine&) = delete;
    Engine& operator=(const Engine&) = delete;

    py::dict run(const std::string& command, const py::dict& data) {
        if (command == "variables") {
            size_t count = 0;
            check(kge_variable_count(engine_, &count));
            py::list variables;
            for (size_t i = 0; i < count; ++i) {
                const char* name = nullptr;
                int dtype = 0, rank = 0;
                size_t shape[4] = {0, 0, 0, 0};
                check(kge_variable_info(engine_, i, &name, &dtype, &rank, shape));
                py::list dims;
                for (int d = 0; d < rank; ++d) dims.append(shape[d]);
                variables.append(py::make_tuple(std::string(name), dims));
            }
            py::dict out;
            out["variables"] = variables;
            return out;
        }
        std::list<std::string> names;
        std::list<std::vector<size_t>> shapes;
        std::vector<kge_array> arrays;
        std::string variable;
        bool has_variable = false;
        for (auto item : data) {
            const std::string key = py::str(item.first);
            if (py::isinstance<py::array>(item.second)) {
                py::array a = py::reinterpret_borrow<py::array>(item.second);
                if (!(a.flags() & py::array::c_style)) throw py::value_error("'" + key + "' must be a C-contiguous array");
                int dtype;
                if (a.dtype().is(py::dtype::of<float>())) dtype = KGE_F32;
                else if (a.dtype().is(py::dtype::of<uint32_t>())) dtype = KGE_U32;
                else if (a.dtype().is(py::dtype::of<int16_t>()) || a.dtype().is(py::dtype("float16"))) dtype = KGE_F16;  // src/lib.cpp:25-35
                else throw py::value_error("'" + key + "' has an element type other than float32, uint32, float16");
                names.push_back(key);
                shapes.emplace_back(a.shape(), a.shape() + a.ndim());
                if (!a.writeable() && (key == "loss" || key == "value" || key == "read_data" || key == "predict_scores" ||
                                       key == "predict_indices"))
                    throw py::value_error("'" + key + "' is written by this command and must be writeable");
                arrays.push_back({names.back().c_str(), dtype, (int)a.ndim(), shapes.back().data(), const_cast<void*>(a.data())});
            } else if (key == "name" && py::isinstance<py::str>(item.second)) {
                variable = item.second.cast<std::string>();
                has_variable = true;
            }
        }
        int status;
        {
            py::gil_scoped_release release;
            status = kge_run(engine_, command.c_str(), arrays.data(), arrays.size(), has_variable ? variable.c_str() : nullptr);
        }
        check(status);
        return py::dict();
    }

    // Multi-process set-up and the device-resident training path (see include/kge_b200.h).
    py::bytes comm_export() {
        std::string buf(kge_comm_handle_bytes(), '\0');
        check(kge_comm_export(engine_, &buf[0]));
        return py::bytes(buf);
    }
    void comm_connect(const py::bytes& all_handles, size_t world_size) {
        const std::string buf = all_handles;
        if (buf.size() != world_size * kge_comm_handle_bytes()) throw py::value_error("comm_connect: wrong handle buffer size");
        check(kge_comm_connect(engine_, buf.data(), world_size));
    }
    py::tuple last_run_stats() {
        float ms = 0.f;
        unsigned long long launches = 0;
        check(kge_last_run_stats(engine_, &ms, &launches));
        return py::make_tuple(ms, launches);
    }

   private:
    void check(int status) {
        if (status != KGE_OK) raise(status, kge_last_error(engine_));
    }
    kge_engine* engine_ = nullptr;
};

}  // namespace

PYBIND11_MODULE(libpoplar_kge, m) {
    m.doc() = "BESS knowledge-graph-embedding engine on B200: the low-level Engine(settings, gp_folder).run(command, data)";
    py::class_<Engine>(m, "Engine", "Allocate the shard tables and per-step buffers on the GPU")
        .def(py::init<const py::dict&, const std::string&>(), py::arg("settings"), py::arg("gp_folder"))
        .def("run", &Engine::run, "Execute a command", py::arg("command"), py::arg("data"))
        .def("comm_export", &Engine::comm_export)
        .def("comm_connect", &Engine::comm_connect, py::arg("all_handles"), py::arg("world_size"))
        .def("last_run_stats", &Engine::last_run_stats);
}
