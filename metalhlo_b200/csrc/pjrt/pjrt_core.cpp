// PJRT plugin entry point, error and event objects (reference: Sources/PJRTMetalHLO/PJRTApi.swift:15-170,
// PJRTError.swift, PJRTEvent.swift).
#include <cstdio>

#include "pjrt_objects.h"

namespace pjrt_b200 {

PJRT_Error* make_error(PJRT_Error_Code code, const std::string& message) { return new PJRT_Error{code, message}; }

PJRT_Error* unimplemented(const char* function_name) {
    return make_error(PJRT_Error_Code_UNIMPLEMENTED, std::string(function_name) + " is not implemented");
}

PJRT_Event* new_ready_event() { return new PJRT_Event(); }
PJRT_Event* new_pending_event() {
    PJRT_Event* e = new PJRT_Event();
    e->ready = false;
    e->refs.store(2, std::memory_order_relaxed);  // the caller's reference and the producer's, dropped by event_complete()
    return e;
}
void event_complete(PJRT_Event* e) {
    std::vector<std::pair<PJRT_Event_OnReadyCallback, void*>> callbacks;
    {
        std::lock_guard<std::mutex> lock(e->mu);
        e->ready = true;
        callbacks.swap(e->callbacks);
    }
    e->cv.notify_all();
    for (auto& cb : callbacks) cb.first(nullptr, cb.second);
    event_release(e);
}
void event_retain(PJRT_Event* e) { e->refs.fetch_add(1, std::memory_order_relaxed); }
void event_release(PJRT_Event* e) {
    if (e && e->refs.fetch_sub(1, std::memory_order_acq_rel) == 1) delete e;
}

// FNV-1a over the program text: a stable fingerprint across processes (the reference hashes the text with a
// per-process seeded hasher, PJRTExecutable.swift:330-340; a stable value is a superset of that contract).
std::string hex_hash(const std::string& text) {
    uint64_t h = 1469598103934665603ull;
    for (unsigned char c : text) {
        h ^= c;
        h *= 1099511628211ull;
    }
    char buf[17];
    snprintf(buf, sizeof buf, "%016llx", static_cast<unsigned long long>(h));
    return buf;
}

namespace {

// ---- errors (PJRTError.swift:27-68) ----
void error_destroy(PJRT_Error_Destroy_Args* args) {
    if (args && args->error) delete args->error;
}

void error_message(PJRT_Error_Message_Args* args) {
    if (!args) return;
    if (!args->error) {
        args->message = "";
        args->message_size = 0;
        return;
    }
    args->message = args->error->message.c_str();
    args->message_size = args->error->message.size();
}

PJRT_Error* error_get_code(PJRT_Error_GetCode_Args* args) {
    PJRT_B200_REQUIRE(args, "NULL args");
    PJRT_B200_REQUIRE(args->error, "NULL error");
    args->code = args->error->code;
    return nullptr;
}

// ---- plugin (PJRTClient.swift:91-110) ----
PJRT_Error* plugin_initialize(PJRT_Plugin_Initialize_Args*) { return nullptr; }

PJRT_Error* plugin_attributes(PJRT_Plugin_Attributes_Args* args) {
    PJRT_B200_REQUIRE(args, "NULL args");
    args->attributes = nullptr;
    args->num_attributes = 0;
    return nullptr;
}

// ---- events (PJRTEvent.swift:104-166) ----
PJRT_Error* copy_error(const PJRT_Error* e) { return e ? new PJRT_Error{e->code, e->message} : nullptr; }

PJRT_Error* event_destroy(PJRT_Event_Destroy_Args* args) {
    if (args && args->event) event_release(args->event);
    return nullptr;
}

PJRT_Error* event_is_ready(PJRT_Event_IsReady_Args* args) {
    PJRT_B200_REQUIRE(args && args->event, "NULL args or event");
    std::lock_guard<std::mutex> lock(args->event->mu);
    args->is_ready = args->event->ready;
    return nullptr;
}

PJRT_Error* event_error(PJRT_Event_Error_Args* args) {
    PJRT_B200_REQUIRE(args && args->event, "NULL args or event");
    std::lock_guard<std::mutex> lock(args->event->mu);
    return copy_error(args->event->error.get());
}

// Execution and host-to-device transfers are synchronous, so their events are complete on creation; the event of a
// device-to-host transfer is pending until the copy stream's completion function has run (event_complete).
PJRT_Error* event_await(PJRT_Event_Await_Args* args) {
    PJRT_B200_REQUIRE(args && args->event, "NULL args or event");
    std::unique_lock<std::mutex> lock(args->event->mu);
    args->event->cv.wait(lock, [&] { return args->event->ready; });
    return copy_error(args->event->error.get());
}

PJRT_Error* event_on_ready(PJRT_Event_OnReady_Args* args) {
    PJRT_B200_REQUIRE(args && args->event, "NULL args or event");
    PJRT_B200_REQUIRE(args->callback, "NULL callback");
    PJRT_Error* err = nullptr;
    {
        std::lock_guard<std::mutex> lock(args->event->mu);
        if (!args->event->ready) {
            args->event->callbacks.emplace_back(args->callback, args->user_arg);
            return nullptr;
        }
        err = copy_error(args->event->error.get());
    }
    args->callback(err, args->user_arg);  // the callback owns err
    return nullptr;
}

}  // namespace

void fill_core_api(PJRT_Api* api) {
    api->PJRT_Error_Destroy = error_destroy;
    api->PJRT_Error_Message = error_message;
    api->PJRT_Error_GetCode = error_get_code;
    api->PJRT_Plugin_Initialize = plugin_initialize;
    api->PJRT_Plugin_Attributes = plugin_attributes;
    api->PJRT_Event_Destroy = event_destroy;
    api->PJRT_Event_IsReady = event_is_ready;
    api->PJRT_Event_Error = event_error;
    api->PJRT_Event_Await = event_await;
    api->PJRT_Event_OnReady = event_on_ready;
}

}  // namespace pjrt_b200

// The one exported symbol (PJRTApi.swift:15-21). The table is built once; entries the plugin does not implement stay
// NULL, as in the reference, and callers probe them before use.
extern "C" __attribute__((visibility("default"))) const PJRT_Api* GetPjrtApi(void) {
    static PJRT_Api api = [] {
        PJRT_Api a;
        std::memset(&a, 0, sizeof a);
        a.struct_size = PJRT_Api_STRUCT_SIZE;
        a.extension_start = nullptr;
        a.pjrt_api_version.struct_size = PJRT_Api_Version_STRUCT_SIZE;
        a.pjrt_api_version.extension_start = nullptr;
        a.pjrt_api_version.major_version = PJRT_API_MAJOR;
        a.pjrt_api_version.minor_version = PJRT_API_MINOR;
        pjrt_b200::fill_core_api(&a);
        pjrt_b200::fill_client_api(&a);
        pjrt_b200::fill_buffer_api(&a);
        pjrt_b200::fill_executable_api(&a);
        return a;
    }();
    return &api;
}
