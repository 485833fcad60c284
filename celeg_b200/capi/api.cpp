// The C interface of include/celeg_b200/api.h. Counterpart in celeg: src/api/engine.cpp, options.cpp and
// api_common.cpp (a C face over its C++ engine, errors caught at the boundary and kept per engine).
//
// Here the engine's host side (configuration, cache accounting, scheduler) is the Python package
// celeg_b200, and this file is the C face over it: it finds or starts a Python interpreter, imports
// celeg_b200.capi.bridge, and turns every call into one call of a bridge function with plain values. All
// device work stays in the kernel library that the package loads. Any thread may call: each call takes the
// interpreter lock for its duration (the bridge releases it while it waits for the GPU).
#define PY_SSIZE_T_CLEAN
#include <Python.h>

#include <dlfcn.h>

#include <cstdarg>
#include <cstring>
#include <mutex>
#include <string>

#include "../../include/celeg_b200/api.h"

struct celeg_b200_engine {
    PyObject* object = nullptr;      // celeg_b200.engine.engine.Engine
    std::string error;
};

namespace {

std::mutex g_start_mutex;
bool g_started_here = false;
PyObject* g_bridge = nullptr;        // celeg_b200.capi.bridge, kept for the life of the process
thread_local std::string g_create_error;

// The folder that holds the celeg_b200 package: this library lives in <root>/celeg_b200/capi/_build/.
std::string package_root() {
    Dl_info info;
    if (dladdr(reinterpret_cast<void*>(&package_root), &info) == 0 || info.dli_fname == nullptr) return "";
    std::string path(info.dli_fname);
    for (int up = 0; up < 4; ++up) {
        const size_t slash = path.find_last_of('/');
        if (slash == std::string::npos) return "";
        path.erase(slash);
    }
    return path;
}

// The message of the pending Python exception (cleared), and its status code.
celeg_b200_status take_exception(std::string& message) {
    PyObject *type = nullptr, *value = nullptr, *trace = nullptr;
    PyErr_Fetch(&type, &value, &trace);
    PyErr_NormalizeException(&type, &value, &trace);
    celeg_b200_status code = CELEG_B200_STATUS_ERROR;
    message = "unknown error";
    if (value != nullptr) {
        if (PyObject* text = PyObject_Str(value)) {
            if (const char* utf8 = PyUnicode_AsUTF8(text)) {
                const char* name = type ? reinterpret_cast<PyTypeObject*>(type)->tp_name : "Exception";
                message = std::string(name) + ": " + utf8;
            }
            Py_DECREF(text);
        }
        if (g_bridge != nullptr) {
            if (PyObject* result = PyObject_CallMethod(g_bridge, "classify", "O", value)) {
                const long number = PyLong_AsLong(result);
                if (number >= 1 && number <= 5) code = static_cast<celeg_b200_status>(number);
                Py_DECREF(result);
            }
            PyErr_Clear();
        }
    }
    Py_XDECREF(type);
    Py_XDECREF(value);
    Py_XDECREF(trace);
    return code;
}

// Holds the interpreter lock for its lifetime; starts an interpreter first if the process has none.
class Interpreter {
public:
    Interpreter() {
        {
            std::lock_guard<std::mutex> lock(g_start_mutex);
            if (!Py_IsInitialized()) {
                Py_InitializeEx(0);
                g_started_here = true;
                PyEval_SaveThread();             // leave the interpreter unlocked between calls
            }
        }
        state_ = PyGILState_Ensure();
    }
    ~Interpreter() { PyGILState_Release(state_); }
    Interpreter(const Interpreter&) = delete;
    Interpreter& operator=(const Interpreter&) = delete;

    // celeg_b200.capi.bridge; null with a Python exception pending if it cannot be imported
    PyObject* bridge() {
        if (g_bridge != nullptr) return g_bridge;
        const std::string root = package_root();
        if (!root.empty()) {
            PyObject* sys_path = PySys_GetObject("path");          // borrowed
            PyObject* entry = PyUnicode_FromString(root.c_str());
            if (sys_path != nullptr && entry != nullptr && PySequence_Contains(sys_path, entry) == 0)
                PyList_Insert(sys_path, 0, entry);
            Py_XDECREF(entry);
        }
#ifdef CELEG_B200_SITE_PACKAGES
        if (g_started_here) {
            // an interpreter started here knows the system's modules only: add the folders the package's own
            // interpreter had at build time (where torch lives), separated by ':'
            PyObject* sys_path = PySys_GetObject("path");
            std::string folders(CELEG_B200_SITE_PACKAGES);
            size_t begin = 0;
            while (sys_path != nullptr && begin <= folders.size()) {
                const size_t end = folders.find(':', begin);
                const std::string folder = folders.substr(begin, end == std::string::npos ? std::string::npos : end - begin);
                if (!folder.empty()) {
                    PyObject* entry = PyUnicode_FromString(folder.c_str());
                    if (entry != nullptr && PySequence_Contains(sys_path, entry) == 0) PyList_Append(sys_path, entry);
                    Py_XDECREF(entry);
                }
                if (end == std::string::npos) break;
                begin = end + 1;
            }
        }
#endif
        g_bridge = PyImport_ImportModule("celeg_b200.capi.bridge");
        return g_bridge;
    }

private:
    PyGILState_STATE state_;
};

celeg_b200_status fail(celeg_b200_engine* engine, celeg_b200_status code, const char* message) {
    if (engine != nullptr) engine->error = message;
    return code;
}

// Calls bridge.<name>(engine, *arguments) and hands the result to `use`. `format` is a Py_BuildValue format
// in parentheses (so that it builds a tuple), or "" for no further arguments. Exceptions become a status and
// the engine's error text.
template <typename Use>
celeg_b200_status call(celeg_b200_engine* engine, const char* name, Use use, const char* format, ...) {
    if (engine == nullptr || engine->object == nullptr) return CELEG_B200_STATUS_INVALID_ARGUMENT;
    Interpreter python;
    PyObject* bridge = python.bridge();
    if (bridge == nullptr) return take_exception(engine->error);
    PyObject* function = PyObject_GetAttrString(bridge, name);
    if (function == nullptr) return take_exception(engine->error);
    PyObject* extra = nullptr;
    if (format[0] != 0) {
        va_list arguments;
        va_start(arguments, format);
        extra = Py_VaBuildValue(format, arguments);
        va_end(arguments);
        if (extra == nullptr || !PyTuple_Check(extra)) {
            Py_XDECREF(extra);
            Py_DECREF(function);
            if (!PyErr_Occurred()) PyErr_SetString(PyExc_SystemError, "arguments of a bridge call must build a tuple");
            return take_exception(engine->error);
        }
    }
    const Py_ssize_t extras = extra != nullptr ? PyTuple_GET_SIZE(extra) : 0;
    PyObject* tuple = PyTuple_New(1 + extras);
    if (tuple != nullptr) {
        Py_INCREF(engine->object);
        PyTuple_SET_ITEM(tuple, 0, engine->object);
        for (Py_ssize_t i = 0; i < extras; ++i) {
            PyObject* item = PyTuple_GET_ITEM(extra, i);
            Py_INCREF(item);
            PyTuple_SET_ITEM(tuple, 1 + i, item);
        }
    }
    Py_XDECREF(extra);
    PyObject* result = tuple != nullptr ? PyObject_CallObject(function, tuple) : nullptr;
    Py_XDECREF(tuple);
    Py_DECREF(function);
    if (result == nullptr) return take_exception(engine->error);
    celeg_b200_status status = use(result);
    Py_DECREF(result);
    if (PyErr_Occurred()) {
        const celeg_b200_status raised = take_exception(engine->error);
        return status != CELEG_B200_STATUS_OK ? status : raised;
    }
    return status;
}

celeg_b200_status nothing(PyObject*) { return CELEG_B200_STATUS_OK; }

}  // namespace

extern "C" {

void celeg_b200_engine_options_init(celeg_b200_engine_options* options) {
    if (options == nullptr) return;
    std::memset(options, 0, sizeof(*options));
    options->struct_size = sizeof(*options);
    options->cuda_graph = 1;
    options->max_active_requests = 8;
    options->max_batched_tokens = 512;
    options->prefill_chunk_tokens = 256;
    options->page_tokens = 16;
}

void celeg_b200_request_options_init(celeg_b200_request_options* options) {
    if (options == nullptr) return;
    std::memset(options, 0, sizeof(*options));
    options->struct_size = sizeof(*options);
    options->max_new_tokens = 128;
    options->eos_token_id = -1;
    options->generation.struct_size = sizeof(options->generation);
    options->generation.temperature = 0.1f;
    options->generation.top_k = 50;
    options->generation.top_p = 1.0f;
    options->generation.repetition_penalty = 1.05f;
    options->generation.seed = 1;
}

celeg_b200_engine* celeg_b200_engine_create(const char* model_path, const celeg_b200_engine_options* options) {
    if (model_path == nullptr || *model_path == 0 || options == nullptr) {
        g_create_error = "a model path and options are required";
        return nullptr;
    }
    if (options->struct_size < sizeof(*options)) {
        g_create_error = "engine options are smaller than this library's struct: fill them with "
                         "celeg_b200_engine_options_init of the same library";
        return nullptr;
    }
    Interpreter python;
    PyObject* bridge = python.bridge();
    if (bridge == nullptr) {
        take_exception(g_create_error);
        return nullptr;
    }
    PyObject* object = PyObject_CallMethod(
        bridge, "create", "siiiiiiiiKi", model_path, (int)options->max_context, (int)options->dtype,
        (int)options->device, (int)options->cuda_graph, (int)options->max_active_requests,
        (int)options->max_batched_tokens, (int)options->prefill_chunk_tokens, (int)options->page_tokens,
        (unsigned long long)options->logical_kv_pages, (int)options->scheduler_policy);
    if (object == nullptr) {
        take_exception(g_create_error);
        return nullptr;
    }
    celeg_b200_engine* engine = new celeg_b200_engine();
    engine->object = object;
    return engine;
}

void celeg_b200_engine_destroy(celeg_b200_engine* engine) {
    if (engine == nullptr) return;
    if (engine->object != nullptr) {
        call(engine, "destroy", nothing, "");
        Interpreter python;
        Py_CLEAR(engine->object);
    }
    delete engine;
}

celeg_b200_status celeg_b200_engine_submit(celeg_b200_engine* engine, const int32_t* tokens, size_t count,
                                           const celeg_b200_request_options* options,
                                           celeg_b200_request_id* request_id) {
    if (engine == nullptr) return CELEG_B200_STATUS_INVALID_ARGUMENT;
    if (tokens == nullptr || count == 0 || options == nullptr || request_id == nullptr)
        return fail(engine, CELEG_B200_STATUS_INVALID_ARGUMENT, "tokens, options and a place for the id are required");
    if (options->struct_size < sizeof(*options) || options->generation.struct_size < sizeof(options->generation))
        return fail(engine, CELEG_B200_STATUS_INVALID_ARGUMENT,
                    "request options are smaller than this library's struct: fill them with "
                    "celeg_b200_request_options_init of the same library");
    PyObject* list = nullptr;
    {
        Interpreter python;
        list = PyList_New((Py_ssize_t)count);
        if (list == nullptr) return take_exception(engine->error);
        for (size_t i = 0; i < count; ++i) PyList_SET_ITEM(list, (Py_ssize_t)i, PyLong_FromLong(tokens[i]));
    }
    const celeg_b200_status status = call(
        engine, "submit",
        [&](PyObject* result) {
            const unsigned long long id = PyLong_AsUnsignedLongLong(result);
            if (PyErr_Occurred()) return CELEG_B200_STATUS_ERROR;
            *request_id = id;
            return CELEG_B200_STATUS_OK;
        },
        "(OIiififfK)", list, (unsigned int)options->max_new_tokens, (int)options->eos_token_id, (int)options->priority,
        (double)options->generation.temperature, (int)options->generation.top_k, (double)options->generation.top_p,
        (double)options->generation.repetition_penalty, (unsigned long long)options->generation.seed);
    {
        Interpreter python;
        Py_DECREF(list);
    }
    return status;
}

celeg_b200_status celeg_b200_engine_poll(celeg_b200_engine* engine, celeg_b200_request_id request_id, int32_t* output,
                                         size_t capacity, size_t* count, int* finished) {
    if (engine == nullptr) return CELEG_B200_STATUS_INVALID_ARGUMENT;
    if (output == nullptr || capacity == 0 || count == nullptr || finished == nullptr)
        return fail(engine, CELEG_B200_STATUS_INVALID_ARGUMENT, "an output buffer and places for count and finished are required");
    return call(
        engine, "poll",
        [&](PyObject* result) {
            PyObject* tokens = PyTuple_GetItem(result, 0);          // borrowed
            PyObject* done = PyTuple_GetItem(result, 1);
            if (tokens == nullptr || done == nullptr) return CELEG_B200_STATUS_ERROR;
            const Py_ssize_t n = PyList_Size(tokens);
            if (n < 0 || (size_t)n > capacity) return CELEG_B200_STATUS_BUFFER_TOO_SMALL;
            for (Py_ssize_t i = 0; i < n; ++i) output[i] = (int32_t)PyLong_AsLong(PyList_GET_ITEM(tokens, i));
            *count = (size_t)n;
            *finished = PyObject_IsTrue(done) ? 1 : 0;
            return CELEG_B200_STATUS_OK;
        },
        "(Kn)", (unsigned long long)request_id, (Py_ssize_t)capacity);
}

celeg_b200_status celeg_b200_engine_status(celeg_b200_engine* engine, celeg_b200_request_id request_id,
                                           celeg_b200_request_status* status) {
    if (engine == nullptr || status == nullptr) return CELEG_B200_STATUS_INVALID_ARGUMENT;
    return call(
        engine, "status",
        [&](PyObject* result) {
            *status = static_cast<celeg_b200_request_status>(PyLong_AsLong(result));
            return CELEG_B200_STATUS_OK;
        },
        "(K)", (unsigned long long)request_id);
}

celeg_b200_status celeg_b200_engine_cancel(celeg_b200_engine* engine, celeg_b200_request_id request_id) {
    return call(engine, "cancel", nothing, "(K)", (unsigned long long)request_id);
}

celeg_b200_status celeg_b200_engine_release(celeg_b200_engine* engine, celeg_b200_request_id request_id) {
    return call(engine, "release", nothing, "(K)", (unsigned long long)request_id);
}

celeg_b200_status celeg_b200_engine_step(celeg_b200_engine* engine, int* progressed) {
    if (engine == nullptr || progressed == nullptr) return CELEG_B200_STATUS_INVALID_ARGUMENT;
    return call(engine, "step", [&](PyObject* result) {
        *progressed = PyObject_IsTrue(result) ? 1 : 0;
        return CELEG_B200_STATUS_OK;
    }, "");
}

celeg_b200_status celeg_b200_engine_start(celeg_b200_engine* engine) { return call(engine, "start", nothing, ""); }

celeg_b200_status celeg_b200_engine_stop(celeg_b200_engine* engine) { return call(engine, "stop", nothing, ""); }

celeg_b200_status celeg_b200_engine_get_metrics(celeg_b200_engine* engine, celeg_b200_metrics* metrics) {
    if (engine == nullptr || metrics == nullptr) return CELEG_B200_STATUS_INVALID_ARGUMENT;
    if (metrics->struct_size < sizeof(*metrics))
        return fail(engine, CELEG_B200_STATUS_INVALID_ARGUMENT, "set metrics.struct_size to sizeof(celeg_b200_metrics)");
    return call(engine, "metrics", [&](PyObject* result) {
        unsigned long long u[13];
        double ttft = 0, itl = 0, host = 0, gpu = 0;
        unsigned long long ttft_n = 0, itl_n = 0;
        if (!PyArg_ParseTuple(result, "KKKKKKKKKKKKKdKdKdd", &u[0], &u[1], &u[2], &u[3], &u[4], &u[5], &u[6], &u[7],
                              &u[8], &u[9], &u[10], &u[11], &u[12], &ttft, &ttft_n, &itl, &itl_n, &host, &gpu))
            return CELEG_B200_STATUS_ERROR;
        metrics->submitted = u[0]; metrics->completed = u[1]; metrics->cancelled = u[2]; metrics->failed = u[3];
        metrics->preempted = u[4]; metrics->steps = u[5]; metrics->prefill_tokens = u[6]; metrics->decode_tokens = u[7];
        metrics->active_requests = u[8]; metrics->queued_requests = u[9]; metrics->pages_used = u[10];
        metrics->pages_total = u[11]; metrics->pages_high_water = u[12];
        metrics->ttft_ms_sum = ttft; metrics->ttft_samples = ttft_n; metrics->itl_ms_sum = itl;
        metrics->itl_samples = itl_n; metrics->host_ms_sum = host; metrics->gpu_ms_sum = gpu;
        return CELEG_B200_STATUS_OK;
    }, "");
}

celeg_b200_status celeg_b200_engine_fingerprint(celeg_b200_engine* engine, char* output, size_t capacity) {
    if (engine == nullptr || output == nullptr) return CELEG_B200_STATUS_INVALID_ARGUMENT;
    return call(engine, "fingerprint", [&](PyObject* result) {
        Py_ssize_t length = 0;
        const char* text = PyUnicode_AsUTF8AndSize(result, &length);
        if (text == nullptr) return CELEG_B200_STATUS_ERROR;
        if ((size_t)length + 1 > capacity) return CELEG_B200_STATUS_BUFFER_TOO_SMALL;
        std::memcpy(output, text, (size_t)length + 1);
        return CELEG_B200_STATUS_OK;
    }, "");
}

const char* celeg_b200_engine_last_error(const celeg_b200_engine* engine) {
    return engine != nullptr ? engine->error.c_str() : g_create_error.c_str();
}

}  // extern "C"
