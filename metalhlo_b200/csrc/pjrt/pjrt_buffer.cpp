// PJRT buffer entries and host<->device transfers (reference: Sources/PJRTMetalHLO/PJRTBuffer.swift).
// A PJRT buffer owns one MHLOBufferRef: dense row-major device memory. Transfers are synchronous, so every event
// returned here is already complete.
#include <algorithm>

#include "mhlo_cuda.h"
#include "pjrt_objects.h"

namespace pjrt_b200 {

bool to_mhlo_type(PJRT_Buffer_Type t, MHLOElementType* out) {
    switch (t) {
        case PJRT_Buffer_Type_F16: *out = MHLO_F16; return true;
        case PJRT_Buffer_Type_F32: *out = MHLO_F32; return true;
        case PJRT_Buffer_Type_F64: *out = MHLO_F64; return true;
        case PJRT_Buffer_Type_BF16: *out = MHLO_BF16; return true;
        case PJRT_Buffer_Type_PRED: *out = MHLO_I1; return true;
        case PJRT_Buffer_Type_S8: *out = MHLO_I8; return true;
        case PJRT_Buffer_Type_S16: *out = MHLO_I16; return true;
        case PJRT_Buffer_Type_S32: *out = MHLO_I32; return true;
        case PJRT_Buffer_Type_S64: *out = MHLO_I64; return true;
        case PJRT_Buffer_Type_U8: *out = MHLO_UI8; return true;
        case PJRT_Buffer_Type_U16: *out = MHLO_UI16; return true;
        case PJRT_Buffer_Type_U32: *out = MHLO_UI32; return true;
        case PJRT_Buffer_Type_U64: *out = MHLO_UI64; return true;
        default: return false;
    }
}

PJRT_Buffer_Type from_mhlo_type(MHLOElementType t) {
    switch (t) {
        case MHLO_F16: return PJRT_Buffer_Type_F16;
        case MHLO_F32: return PJRT_Buffer_Type_F32;
        case MHLO_F64: return PJRT_Buffer_Type_F64;
        case MHLO_BF16: return PJRT_Buffer_Type_BF16;
        case MHLO_I1: return PJRT_Buffer_Type_PRED;
        case MHLO_I8: return PJRT_Buffer_Type_S8;
        case MHLO_I16: return PJRT_Buffer_Type_S16;
        case MHLO_I32: return PJRT_Buffer_Type_S32;
        case MHLO_I64: return PJRT_Buffer_Type_S64;
        case MHLO_UI8: return PJRT_Buffer_Type_U8;
        case MHLO_UI16: return PJRT_Buffer_Type_U16;
        case MHLO_UI32: return PJRT_Buffer_Type_U32;
        case MHLO_UI64: return PJRT_Buffer_Type_U64;
    }
    return PJRT_Buffer_Type_INVALID;
}

// Predicates occupy one byte per element in host and device memory; mhlo_element_type_size reports 0 for them.
size_t storage_bytes_per_element(MHLOElementType t) {
    const size_t n = mhlo_element_type_size(t);
    return n ? n : 1;
}

PJRT_Buffer* wrap_buffer(PJRT_Client* client, MHLOBufferRef ref, PJRT_Device* device) {
    auto* b = new PJRT_Buffer();
    b->client = client;
    b->device = device ? device : (client && !client->devices.empty() ? client->devices[0] : nullptr);
    b->mhlo = ref;
    const int32_t rank = mhlo_buffer_rank(ref);
    b->dims.resize(static_cast<size_t>(rank));
    int32_t r = 0;
    mhlo_buffer_shape(ref, b->dims.data(), &r);
    b->type = from_mhlo_type(mhlo_buffer_element_type(ref));
    b->bytes = mhlo_buffer_byte_count(ref);
    for (int i = rank - 1; i >= 0; --i) b->minor_to_major.push_back(i);
    b->ready = new_ready_event();
    if (client) {
        const int64_t now = client->live_buffer_bytes.fetch_add(static_cast<int64_t>(b->bytes)) + static_cast<int64_t>(b->bytes);
        int64_t peak = client->peak_buffer_bytes.load();
        while (now > peak && !client->peak_buffer_bytes.compare_exchange_weak(peak, now)) {}
        client->num_allocs.fetch_add(1);
    }
    return b;
}

void present_as_complex(PJRT_Buffer* b) {
    if (b->dims.empty() || b->dims.back() != 2) return;
    if (b->type == PJRT_Buffer_Type_F32) b->type = PJRT_Buffer_Type_C64;
    else if (b->type == PJRT_Buffer_Type_F64) b->type = PJRT_Buffer_Type_C128;
    else return;
    b->dims.pop_back();
    b->minor_to_major.clear();
    for (int i = static_cast<int>(b->dims.size()) - 1; i >= 0; --i) b->minor_to_major.push_back(i);
}

namespace {

void release_storage(PJRT_Buffer* b) {
    if (!b->mhlo) return;
    mhlo_buffer_destroy(b->mhlo);
    b->mhlo = nullptr;
    if (b->client) b->client->live_buffer_bytes.fetch_sub(static_cast<int64_t>(b->bytes));
}

// Copies a strided host tensor into dense row-major order.
void pack_dense(const uint8_t* src, uint8_t* dst, const std::vector<int64_t>& dims, const int64_t* byte_strides, size_t elem) {
    const size_t rank = dims.size();
    std::vector<int64_t> idx(rank, 0);
    int64_t total = 1;
    for (int64_t d : dims) total *= d;
    for (int64_t n = 0; n < total; ++n) {
        int64_t off = 0;
        for (size_t d = 0; d < rank; ++d) off += idx[d] * byte_strides[d];
        std::memcpy(dst + static_cast<size_t>(n) * elem, src + off, elem);
        for (size_t d = rank; d-- > 0;) {
            if (++idx[d] < dims[d]) break;
            idx[d] = 0;
        }
    }
}

// PJRTBuffer.swift:98-148. The data is copied during the call, so done_with_host_buffer is complete on return
// whatever the host-buffer semantics; the zero-copy modes degrade to a copy, which their contract allows.
PJRT_Error* buffer_from_host(PJRT_Client_BufferFromHostBuffer_Args* args) {
    PJRT_B200_REQUIRE(args && args->client, "NULL args or client");
    MHLOElementType et;
    // complex elements are stored as (re, im) pairs of their part type: one more dimension of extent 2 below this layer
    const bool complex_pairs = args->type == PJRT_Buffer_Type_C64 || args->type == PJRT_Buffer_Type_C128;
    const PJRT_Buffer_Type part_type = args->type == PJRT_Buffer_Type_C64 ? PJRT_Buffer_Type_F32 : args->type == PJRT_Buffer_Type_C128 ? PJRT_Buffer_Type_F64 : args->type;
    if (!to_mhlo_type(part_type, &et))
        return make_error(PJRT_Error_Code_INVALID_ARGUMENT, "Unsupported element type: " + std::to_string(static_cast<int>(args->type)));
    std::vector<int64_t> dims;
    if (args->dims) dims.assign(args->dims, args->dims + args->num_dims);
    int64_t count = 1;
    for (int64_t d : dims) {
        if (d < 0) return make_error(PJRT_Error_Code_INVALID_ARGUMENT, "negative dimension");
        count *= d;
    }
    const size_t elem = storage_bytes_per_element(et) * (complex_pairs ? 2 : 1);
    const size_t bytes = static_cast<size_t>(count) * elem;
    PJRT_B200_REQUIRE(args->data || bytes == 0, "NULL data pointer");

    bool dense = true;
    if (args->byte_strides && args->num_byte_strides == dims.size()) {
        int64_t expect = static_cast<int64_t>(elem);
        for (size_t d = dims.size(); d-- > 0;) {
            if (dims[d] != 1 && args->byte_strides[d] != expect) dense = false;
            expect *= dims[d];
        }
    }
    std::vector<uint8_t> packed;
    const void* src = args->data;
    if (!dense && bytes) {
        packed.resize(bytes);
        pack_dense(static_cast<const uint8_t*>(args->data), packed.data(), dims, args->byte_strides, elem);
        src = packed.data();
    }
    // the target: the given device, else the device of the given memory, else device 0
    PJRT_Device* target = args->device;
    if (!target && args->memory && !args->memory->devices.empty()) target = args->memory->devices[0];
    if (!target) target = args->client->devices[0];
    if (target->client != args->client) return make_error(PJRT_Error_Code_INVALID_ARGUMENT, "device belongs to another client");
    MHLOBufferRef ref = nullptr;
    std::vector<int64_t> stored_dims = dims;
    if (complex_pairs) stored_dims.push_back(2);
    const MHLOStatusCode st = mhlo_buffer_create(target->mhlo, src, bytes, stored_dims.data(), static_cast<int32_t>(stored_dims.size()), et, &ref);
    if (st != MHLO_OK || !ref)
        return make_error(PJRT_Error_Code_INTERNAL, std::string("Buffer creation failed: ") + mhlo_get_last_error());
    args->done_with_host_buffer = new_ready_event();
    args->buffer = wrap_buffer(args->client, ref, target);
    if (complex_pairs) present_as_complex(args->buffer);
    return nullptr;
}

PJRT_Error* buffer_destroy(PJRT_Buffer_Destroy_Args* args) {
    if (!args || !args->buffer) return nullptr;
    release_storage(args->buffer);
    event_release(args->buffer->ready);
    delete args->buffer;
    return nullptr;
}

PJRT_Error* buffer_element_type(PJRT_Buffer_ElementType_Args* args) {
    PJRT_B200_REQUIRE(args && args->buffer, "NULL args");
    args->type = args->buffer->type;
    return nullptr;
}

PJRT_Error* buffer_dimensions(PJRT_Buffer_Dimensions_Args* args) {
    PJRT_B200_REQUIRE(args && args->buffer, "NULL args");
    args->dims = args->buffer->dims.data();
    args->num_dims = args->buffer->dims.size();
    return nullptr;
}

PJRT_Error* buffer_unpadded_dimensions(PJRT_Buffer_UnpaddedDimensions_Args* args) {
    PJRT_B200_REQUIRE(args && args->buffer, "NULL args");
    args->unpadded_dims = args->buffer->dims.data();
    args->num_dims = args->buffer->dims.size();
    return nullptr;
}

PJRT_Error* buffer_dynamic_dimension_indices(PJRT_Buffer_DynamicDimensionIndices_Args* args) {
    PJRT_B200_REQUIRE(args && args->buffer, "NULL args");
    args->dynamic_dim_indices = nullptr;
    args->num_dynamic_dims = 0;
    return nullptr;
}

// Dense row-major, untiled (PJRTBuffer.swift:212-226).
PJRT_Error* buffer_get_memory_layout(PJRT_Buffer_GetMemoryLayout_Args* args) {
    PJRT_B200_REQUIRE(args && args->buffer, "NULL args");
    std::memset(&args->layout, 0, sizeof args->layout);
    args->layout.struct_size = PJRT_Buffer_MemoryLayout_STRUCT_SIZE;
    args->layout.type = PJRT_Buffer_MemoryLayout_Type_Tiled;
    args->layout.tiled.struct_size = PJRT_Buffer_MemoryLayout_Tiled_STRUCT_SIZE;
    args->layout.tiled.minor_to_major = args->buffer->minor_to_major.data();
    args->layout.tiled.minor_to_major_size = args->buffer->minor_to_major.size();
    args->layout.tiled.tile_dims = nullptr;
    args->layout.tiled.tile_dim_sizes = nullptr;
    args->layout.tiled.num_tiles = 0;
    return nullptr;
}

PJRT_Error* buffer_on_device_size(PJRT_Buffer_OnDeviceSizeInBytes_Args* args) {
    PJRT_B200_REQUIRE(args && args->buffer, "NULL args");
    args->on_device_size_in_bytes = args->buffer->bytes;
    return nullptr;
}

PJRT_Error* buffer_device(PJRT_Buffer_Device_Args* args) {
    PJRT_B200_REQUIRE(args && args->buffer && args->buffer->client, "NULL args");
    args->device = args->buffer->device;
    return nullptr;
}

PJRT_Error* buffer_memory(PJRT_Buffer_Memory_Args* args) {
    PJRT_B200_REQUIRE(args && args->buffer && args->buffer->client, "NULL args");
    args->memory = args->buffer->device->memories[0];
    return nullptr;
}

PJRT_Error* buffer_delete(PJRT_Buffer_Delete_Args* args) {
    PJRT_B200_REQUIRE(args && args->buffer, "NULL args");
    release_storage(args->buffer);
    return nullptr;
}

PJRT_Error* buffer_is_deleted(PJRT_Buffer_IsDeleted_Args* args) {
    PJRT_B200_REQUIRE(args && args->buffer, "NULL args");
    args->is_deleted = args->buffer->mhlo == nullptr;
    return nullptr;
}

// Copy into a fresh buffer on `target` (PJRTBuffer.swift:392-440). Same device: one device-to-device copy on that device.
// Another GPU of this client: through pinned-size host memory, which needs no peer mapping between the two devices.
PJRT_Error* duplicate(PJRT_Buffer* src, PJRT_Device* target, PJRT_Buffer** out, const char* what) {
    if (!src->mhlo) return make_error(PJRT_Error_Code_FAILED_PRECONDITION, std::string(what) + ": buffer was deleted");
    if (!target) target = src->device;
    if (target->client != src->client) return make_error(PJRT_Error_Code_INVALID_ARGUMENT, std::string(what) + ": device belongs to another client");
    // shape and type as stored (a complex buffer is a float buffer of pairs, one rank higher)
    const bool complex_pairs = src->type == PJRT_Buffer_Type_C64 || src->type == PJRT_Buffer_Type_C128;
    const MHLOElementType et = mhlo_buffer_element_type(src->mhlo);
    std::vector<int64_t> stored(static_cast<size_t>(mhlo_buffer_rank(src->mhlo)));
    int32_t stored_rank = 0;
    mhlo_buffer_shape(src->mhlo, stored.data(), &stored_rank);
    MHLOBufferRef ref = nullptr;
    if (target != src->device) {
        std::vector<uint8_t> host(src->bytes);
        if (src->bytes && mhlo_buffer_to_host(src->mhlo, host.data(), host.size()) != MHLO_OK)
            return make_error(PJRT_Error_Code_INTERNAL, std::string(what) + " failed: " + mhlo_get_last_error());
        if (mhlo_buffer_create(target->mhlo, host.data(), host.size(), stored.data(), static_cast<int32_t>(stored.size()), et, &ref) != MHLO_OK)
            return make_error(PJRT_Error_Code_INTERNAL, std::string(what) + " failed: " + mhlo_get_last_error());
        *out = wrap_buffer(src->client, ref, target);
        if (complex_pairs) present_as_complex(*out);
        return nullptr;
    }
    if (mhlo_buffer_create_uninitialized(target->mhlo, stored.data(), static_cast<int32_t>(stored.size()), et, &ref) != MHLO_OK)
        return make_error(PJRT_Error_Code_INTERNAL, std::string(what) + " failed: " + mhlo_get_last_error());
    if (src->bytes) {
        int st = mhlo_cuda_device_set(target->cuda_ordinal);
        if (st == MHLO_CUDA_OK) st = mhlo_cuda_copy(mhlo_b200_buffer_device_pointer(ref), mhlo_b200_buffer_device_pointer(src->mhlo), src->bytes, nullptr);
        if (st == MHLO_CUDA_OK) st = mhlo_cuda_stream_sync(nullptr);
        if (st != MHLO_CUDA_OK) {
            mhlo_buffer_destroy(ref);
            return make_error(PJRT_Error_Code_INTERNAL, std::string(what) + " failed: " + mhlo_cuda_last_error());
        }
    }
    *out = wrap_buffer(src->client, ref, target);
    if (complex_pairs) present_as_complex(*out);
    return nullptr;
}

PJRT_Error* buffer_copy_to_device(PJRT_Buffer_CopyToDevice_Args* args) {
    PJRT_B200_REQUIRE(args && args->buffer, "NULL args");
    return duplicate(args->buffer, args->dst_device, &args->dst_buffer, "CopyToDevice");
}

PJRT_Error* buffer_copy_to_memory(PJRT_Buffer_CopyToMemory_Args* args) {
    PJRT_B200_REQUIRE(args && args->buffer, "NULL args");
    PJRT_Device* target = args->dst_memory && !args->dst_memory->devices.empty() ? args->dst_memory->devices[0] : nullptr;
    return duplicate(args->buffer, target, &args->dst_buffer, "CopyToMemory");
}

// PJRTBuffer.swift:270-310: a NULL destination asks for the size only.
PJRT_Error* buffer_to_host(PJRT_Buffer_ToHostBuffer_Args* args) {
    PJRT_B200_REQUIRE(args && args->src, "NULL args");
    PJRT_Buffer* b = args->src;
    if (!args->dst) {
        args->dst_size = b->bytes;
        args->event = new_ready_event();
        return nullptr;
    }
    if (!b->mhlo) return make_error(PJRT_Error_Code_FAILED_PRECONDITION, "ToHostBuffer: buffer was deleted");
    if (args->dst_size < b->bytes)
        return make_error(PJRT_Error_Code_INVALID_ARGUMENT, "ToHostBuffer: destination holds " + std::to_string(args->dst_size) +
                                                                " bytes, buffer needs " + std::to_string(b->bytes));
    args->dst_size = b->bytes;
    if (b->bytes == 0) {
        args->event = new_ready_event();
        return nullptr;
    }
    // the copy runs on the client's transfer stream; the event turns ready from the stream's completion function, so a
    // caller may start the next program before it awaits the bytes
    PJRT_Event* ev = new_pending_event();
    if (mhlo_b200_buffer_to_host_async(b->mhlo, args->dst, b->bytes, [](void* e) { event_complete(static_cast<PJRT_Event*>(e)); }, ev) != MHLO_OK) {
        event_release(ev);
        event_release(ev);
        return make_error(PJRT_Error_Code_INTERNAL, std::string("ToHostBuffer failed: ") + mhlo_get_last_error());
    }
    args->event = ev;
    return nullptr;
}

PJRT_Error* buffer_copy_raw_to_host(PJRT_Buffer_CopyRawToHost_Args* args) {
    PJRT_B200_REQUIRE(args && args->buffer, "NULL args");
    PJRT_B200_REQUIRE(args->dst, "NULL destination");
    PJRT_Buffer* b = args->buffer;
    if (!b->mhlo) return make_error(PJRT_Error_Code_FAILED_PRECONDITION, "CopyRawToHost: buffer was deleted");
    if (args->offset < 0 || args->transfer_size < 0 || static_cast<uint64_t>(args->offset) + static_cast<uint64_t>(args->transfer_size) > b->bytes)
        return make_error(PJRT_Error_Code_OUT_OF_RANGE, "Copy range exceeds buffer size");
    if (args->transfer_size) {
        const char* dev = static_cast<const char*>(mhlo_b200_buffer_device_pointer(b->mhlo)) + args->offset;
        int st = mhlo_cuda_download(args->dst, dev, static_cast<size_t>(args->transfer_size), nullptr);
        if (st == MHLO_CUDA_OK) st = mhlo_cuda_stream_sync(nullptr);
        if (st != MHLO_CUDA_OK) return make_error(PJRT_Error_Code_INTERNAL, std::string("CopyRawToHost failed: ") + mhlo_cuda_last_error());
    }
    args->event = new_ready_event();
    return nullptr;
}

PJRT_Error* buffer_is_on_cpu(PJRT_Buffer_IsOnCpu_Args* args) {
    PJRT_B200_REQUIRE(args && args->buffer, "NULL args");
    args->is_on_cpu = false;
    return nullptr;
}

PJRT_Error* buffer_ready_event(PJRT_Buffer_ReadyEvent_Args* args) {
    PJRT_B200_REQUIRE(args && args->buffer, "NULL args");
    event_retain(args->buffer->ready);
    args->event = args->buffer->ready;
    return nullptr;
}

// The reference withholds raw pointers (PJRTBuffer.swift:366-390: UNIMPLEMENTED). CUDA device addresses are stable
// and meaningful to the caller (DLPack export, custom kernels), so they are given out here.
PJRT_Error* buffer_unsafe_pointer(PJRT_Buffer_UnsafePointer_Args* args) {
    PJRT_B200_REQUIRE(args && args->buffer, "NULL args");
    if (!args->buffer->mhlo) return make_error(PJRT_Error_Code_FAILED_PRECONDITION, "UnsafePointer: buffer was deleted");
    args->buffer_pointer = reinterpret_cast<uintptr_t>(mhlo_b200_buffer_device_pointer(args->buffer->mhlo));
    return nullptr;
}

PJRT_Error* buffer_opaque_pointer(PJRT_Buffer_OpaqueDeviceMemoryDataPointer_Args* args) {
    PJRT_B200_REQUIRE(args && args->buffer, "NULL args");
    if (!args->buffer->mhlo) return make_error(PJRT_Error_Code_FAILED_PRECONDITION, "OpaqueDeviceMemoryDataPointer: buffer was deleted");
    args->device_memory_ptr = mhlo_b200_buffer_device_pointer(args->buffer->mhlo);
    return nullptr;
}

PJRT_Error* buffer_increase_external_refs(PJRT_Buffer_IncreaseExternalReferenceCount_Args* args) {
    PJRT_B200_REQUIRE(args && args->buffer, "NULL args");
    args->buffer->external_refs.fetch_add(1);
    return nullptr;
}

PJRT_Error* buffer_decrease_external_refs(PJRT_Buffer_DecreaseExternalReferenceCount_Args* args) {
    PJRT_B200_REQUIRE(args && args->buffer, "NULL args");
    if (args->buffer->external_refs.load() <= 0) return make_error(PJRT_Error_Code_FAILED_PRECONDITION, "external reference count is already zero");
    args->buffer->external_refs.fetch_sub(1);
    return nullptr;
}

}  // namespace

void fill_buffer_api(PJRT_Api* api) {
    api->PJRT_Client_BufferFromHostBuffer = buffer_from_host;
    api->PJRT_Buffer_Destroy = buffer_destroy;
    api->PJRT_Buffer_ElementType = buffer_element_type;
    api->PJRT_Buffer_Dimensions = buffer_dimensions;
    api->PJRT_Buffer_UnpaddedDimensions = buffer_unpadded_dimensions;
    api->PJRT_Buffer_DynamicDimensionIndices = buffer_dynamic_dimension_indices;
    api->PJRT_Buffer_GetMemoryLayout = buffer_get_memory_layout;
    api->PJRT_Buffer_OnDeviceSizeInBytes = buffer_on_device_size;
    api->PJRT_Buffer_Device = buffer_device;
    api->PJRT_Buffer_Memory = buffer_memory;
    api->PJRT_Buffer_Delete = buffer_delete;
    api->PJRT_Buffer_IsDeleted = buffer_is_deleted;
    api->PJRT_Buffer_CopyToDevice = buffer_copy_to_device;
    api->PJRT_Buffer_CopyToMemory = buffer_copy_to_memory;
    api->PJRT_Buffer_ToHostBuffer = buffer_to_host;
    api->PJRT_Buffer_CopyRawToHost = buffer_copy_raw_to_host;
    api->PJRT_Buffer_IsOnCpu = buffer_is_on_cpu;
    api->PJRT_Buffer_ReadyEvent = buffer_ready_event;
    api->PJRT_Buffer_UnsafePointer = buffer_unsafe_pointer;
    api->PJRT_Buffer_OpaqueDeviceMemoryDataPointer = buffer_opaque_pointer;
    api->PJRT_Buffer_IncreaseExternalReferenceCount = buffer_increase_external_refs;
    api->PJRT_Buffer_DecreaseExternalReferenceCount = buffer_decrease_external_refs;
}

}  // namespace pjrt_b200
