// PJRT client, device, device description, memory and topology entries (reference:
// Sources/PJRTMetalHLO/PJRTClient.swift, PJRTDevice.swift, PJRTMemory.swift, PJRTTopology.swift).
// One client owns one CUDA device (chosen by mhlo_client_create), or the first METALHLO_NUM_GPUS devices of the process,
// each with its own memory space of kind "device".
#include <cstdlib>
#include <string>

#include "pjrt_objects.h"

namespace pjrt_b200 {
namespace {

const char kPlatformName[] = "metalhlo";  // PJRTTopology.swift:106
const char kPlatformVersion[] = "0.1.0";  // PJRTTopology.swift:107

void add_int_attribute(PJRT_DeviceDescription* d, const char* name, int64_t value) {
    d->attr_names.emplace_back(name);
    PJRT_NamedValue v;
    std::memset(&v, 0, sizeof v);
    v.struct_size = PJRT_NamedValue_STRUCT_SIZE;
    v.type = PJRT_NamedValue_kInt64;
    v.int64_value = value;
    v.value_size = 1;
    d->attributes.push_back(v);
    d->attr_strings.emplace_back();
}

void add_string_attribute(PJRT_DeviceDescription* d, const char* name, const std::string& value) {
    d->attr_names.emplace_back(name);
    PJRT_NamedValue v;
    std::memset(&v, 0, sizeof v);
    v.struct_size = PJRT_NamedValue_STRUCT_SIZE;
    v.type = PJRT_NamedValue_kString;
    v.value_size = value.size();
    d->attributes.push_back(v);
    d->attr_strings.push_back(value);
}

// Name and string pointers are patched once every attribute is in place (vector growth moves the strings).
void seal_attributes(PJRT_DeviceDescription* d) {
    for (size_t i = 0; i < d->attributes.size(); ++i) {
        d->attributes[i].name = d->attr_names[i].c_str();
        d->attributes[i].name_size = d->attr_names[i].size();
        if (d->attributes[i].type == PJRT_NamedValue_kString) d->attributes[i].string_value = d->attr_strings[i].c_str();
    }
}

int env_ordinal() {
    for (const char* name : {"METALHLO_DEVICE", "LOCAL_RANK"}) {
        const char* v = std::getenv(name);
        if (v && *v) return std::atoi(v);
    }
    return 0;
}

// How many GPUs the client exposes as PJRT devices: METALHLO_NUM_GPUS = a count or "all"; unset = 1, the reference's
// single device (PJRTClient.swift:180-193).
int wanted_device_count(int visible) {
    const char* v = std::getenv("METALHLO_NUM_GPUS");
    if (!v || !*v) return 1;
    if (std::string(v) == "all") return visible;
    const int n = std::atoi(v);
    return n < 1 ? 1 : (n > visible ? visible : n);
}

// ---- client (PJRTClient.swift:112-259) ----
PJRT_Error* client_create(PJRT_Client_Create_Args* args) {
    PJRT_B200_REQUIRE(args, "NULL args");
    const int visible = mhlo_b200_device_count();
    const int count = wanted_device_count(visible);
    auto c = std::unique_ptr<PJRT_Client>(new PJRT_Client());
    c->platform_name = kPlatformName;
    c->platform_version = kPlatformVersion;
    const char* policy = std::getenv("METALHLO_DEVICE_POLICY");
    for (int i = 0; i < count; ++i) {
        MHLOClientRef ref = nullptr;
        // one device: the C API's own choice (METALHLO_DEVICE / LOCAL_RANK); several: GPUs 0 .. count-1 of this process
        const MHLOStatusCode st = count == 1 ? mhlo_client_create(&ref) : mhlo_b200_client_create_on_device(i, &ref);
        if (st != MHLO_OK || !ref) {
            const std::string why = mhlo_get_last_error() ? mhlo_get_last_error() : "unknown error";
            for (auto& d : c->owned_devices) mhlo_client_destroy(d->mhlo);
            return make_error(PJRT_Error_Code_INTERNAL, "Failed to create CUDA client: " + why);
        }
        char* name = mhlo_client_device_name(ref);
        const std::string device_name = name ? name : "CUDA device";
        if (name) mhlo_free_string(name);
        std::unique_ptr<PJRT_Device> dev(new PJRT_Device());
        dev->client = c.get();
        dev->index = i;
        dev->cuda_ordinal = count == 1 ? env_ordinal() : i;
        dev->mhlo = ref;
        PJRT_DeviceDescription& d = dev->description;
        d.id = i;
        d.process_index = 0;
        d.kind = "CUDA";
        d.debug_string = "CUDA:" + device_name + (count > 1 ? ":" + std::to_string(i) : "");
        d.to_string = device_name;
        // The two attributes the reference always publishes (PJRTDevice.swift:40-66), then this backend's own.
        add_int_attribute(&d, "ane_available", 0);
        add_string_attribute(&d, "device_policy", policy && *policy ? policy : "auto");
        add_int_attribute(&d, "cuda_ordinal", dev->cuda_ordinal);
        seal_attributes(&d);
        std::unique_ptr<PJRT_Memory> mem(new PJRT_Memory());
        mem->id = i;
        mem->kind_id = 0;
        mem->kind = "device";
        mem->debug_string = "CUDA device memory";
        mem->to_string = "CUDA device";
        mem->devices = {dev.get()};
        dev->memories = {mem.get()};
        c->devices.push_back(dev.get());
        c->memories.push_back(mem.get());
        c->owned_devices.push_back(std::move(dev));
        c->owned_memories.push_back(std::move(mem));
    }
    if (c->devices.empty()) return make_error(PJRT_Error_Code_INTERNAL, "Failed to create CUDA client: No CUDA device available");
    c->mhlo = c->devices[0]->mhlo;
    c->topology.platform_name = kPlatformName;
    c->topology.platform_version = kPlatformVersion;
    for (PJRT_Device* d : c->devices) c->topology.descriptions.push_back(&d->description);
    args->client = c.release();
    return nullptr;
}

PJRT_Error* client_destroy(PJRT_Client_Destroy_Args* args) {
    if (!args || !args->client) return nullptr;
    for (auto& d : args->client->owned_devices) mhlo_client_destroy(d->mhlo);
    delete args->client;
    return nullptr;
}

PJRT_Error* client_platform_name(PJRT_Client_PlatformName_Args* args) {
    PJRT_B200_REQUIRE(args && args->client, "NULL args");
    args->platform_name = args->client->platform_name.c_str();
    args->platform_name_size = args->client->platform_name.size();
    return nullptr;
}

PJRT_Error* client_process_index(PJRT_Client_ProcessIndex_Args* args) {
    PJRT_B200_REQUIRE(args, "NULL args");
    args->process_index = 0;
    return nullptr;
}

PJRT_Error* client_platform_version(PJRT_Client_PlatformVersion_Args* args) {
    PJRT_B200_REQUIRE(args && args->client, "NULL args");
    args->platform_version = args->client->platform_version.c_str();
    args->platform_version_size = args->client->platform_version.size();
    return nullptr;
}

PJRT_Error* client_devices(PJRT_Client_Devices_Args* args) {
    PJRT_B200_REQUIRE(args && args->client, "NULL args");
    args->devices = args->client->devices.data();
    args->num_devices = args->client->devices.size();
    return nullptr;
}

PJRT_Error* client_addressable_devices(PJRT_Client_AddressableDevices_Args* args) {
    PJRT_B200_REQUIRE(args && args->client, "NULL args");
    args->addressable_devices = args->client->devices.data();
    args->num_addressable_devices = args->client->devices.size();
    return nullptr;
}

PJRT_Error* client_lookup_device(PJRT_Client_LookupDevice_Args* args) {
    PJRT_B200_REQUIRE(args && args->client, "NULL args");
    if (args->id < 0 || args->id >= static_cast<int>(args->client->devices.size()))
        return make_error(PJRT_Error_Code_NOT_FOUND, "Device " + std::to_string(args->id) + " not found");
    args->device = args->client->devices[static_cast<size_t>(args->id)];
    return nullptr;
}

PJRT_Error* client_lookup_addressable_device(PJRT_Client_LookupAddressableDevice_Args* args) {
    PJRT_B200_REQUIRE(args && args->client, "NULL args");
    if (args->local_hardware_id < 0 || args->local_hardware_id >= static_cast<int>(args->client->devices.size()))
        return make_error(PJRT_Error_Code_NOT_FOUND, "Local device " + std::to_string(args->local_hardware_id) + " not found");
    args->addressable_device = args->client->devices[static_cast<size_t>(args->local_hardware_id)];
    return nullptr;
}

PJRT_Error* client_addressable_memories(PJRT_Client_AddressableMemories_Args* args) {
    PJRT_B200_REQUIRE(args && args->client, "NULL args");
    args->addressable_memories = args->client->memories.data();
    args->num_addressable_memories = args->client->memories.size();
    return nullptr;
}

PJRT_Error* client_default_device_assignment(PJRT_Client_DefaultDeviceAssignment_Args* args) {
    PJRT_B200_REQUIRE(args, "NULL args");
    const size_t want = static_cast<size_t>(std::max(0, args->num_replicas)) * static_cast<size_t>(std::max(0, args->num_partitions));
    // replica r of a single-partition program runs on device r (all on device 0 when the client exposes only one)
    const size_t n_dev = args->client ? args->client->devices.size() : 1;
    if (args->default_assignment)
        for (size_t i = 0; i < want && i < args->default_assignment_size; ++i)
            args->default_assignment[i] = static_cast<int>(args->num_partitions > 0 ? (i / static_cast<size_t>(args->num_partitions)) % n_dev : 0);
    return nullptr;
}

PJRT_Error* client_topology_description(PJRT_Client_TopologyDescription_Args* args) {
    PJRT_B200_REQUIRE(args && args->client, "NULL args");
    args->topology = &args->client->topology;
    return nullptr;
}

// ---- device descriptions (PJRTDevice.swift:120-195) ----
PJRT_Error* dd_id(PJRT_DeviceDescription_Id_Args* args) {
    PJRT_B200_REQUIRE(args && args->device_description, "NULL args");
    args->id = args->device_description->id;
    return nullptr;
}
PJRT_Error* dd_process_index(PJRT_DeviceDescription_ProcessIndex_Args* args) {
    PJRT_B200_REQUIRE(args && args->device_description, "NULL args");
    args->process_index = args->device_description->process_index;
    return nullptr;
}
PJRT_Error* dd_attributes(PJRT_DeviceDescription_Attributes_Args* args) {
    PJRT_B200_REQUIRE(args && args->device_description, "NULL args");
    args->attributes = args->device_description->attributes.data();
    args->num_attributes = args->device_description->attributes.size();
    return nullptr;
}
PJRT_Error* dd_kind(PJRT_DeviceDescription_Kind_Args* args) {
    PJRT_B200_REQUIRE(args && args->device_description, "NULL args");
    args->device_kind = args->device_description->kind.c_str();
    args->device_kind_size = args->device_description->kind.size();
    return nullptr;
}
PJRT_Error* dd_debug_string(PJRT_DeviceDescription_DebugString_Args* args) {
    PJRT_B200_REQUIRE(args && args->device_description, "NULL args");
    args->debug_string = args->device_description->debug_string.c_str();
    args->debug_string_size = args->device_description->debug_string.size();
    return nullptr;
}
PJRT_Error* dd_to_string(PJRT_DeviceDescription_ToString_Args* args) {
    PJRT_B200_REQUIRE(args && args->device_description, "NULL args");
    args->to_string = args->device_description->to_string.c_str();
    args->to_string_size = args->device_description->to_string.size();
    return nullptr;
}

// ---- devices (PJRTDevice.swift:197-274) ----
PJRT_Error* device_get_description(PJRT_Device_GetDescription_Args* args) {
    PJRT_B200_REQUIRE(args && args->device, "NULL args");
    args->device_description = &args->device->description;
    return nullptr;
}
PJRT_Error* device_is_addressable(PJRT_Device_IsAddressable_Args* args) {
    PJRT_B200_REQUIRE(args && args->device, "NULL args");
    args->is_addressable = true;
    return nullptr;
}
PJRT_Error* device_local_hardware_id(PJRT_Device_LocalHardwareId_Args* args) {
    PJRT_B200_REQUIRE(args && args->device, "NULL args");
    args->local_hardware_id = args->device->index;
    return nullptr;
}
PJRT_Error* device_addressable_memories(PJRT_Device_AddressableMemories_Args* args) {
    PJRT_B200_REQUIRE(args && args->device, "NULL args");
    args->memories = args->device->memories.data();
    args->num_memories = args->device->memories.size();
    return nullptr;
}
PJRT_Error* device_default_memory(PJRT_Device_DefaultMemory_Args* args) {
    PJRT_B200_REQUIRE(args && args->device, "NULL args");
    args->memory = args->device->memories.empty() ? nullptr : args->device->memories[0];
    return nullptr;
}
// The reference reports bytes_in_use = 0 and nothing else; here the bytes held by live PJRT buffers are tracked.
PJRT_Error* device_memory_stats(PJRT_Device_MemoryStats_Args* args) {
    PJRT_B200_REQUIRE(args && args->device, "NULL args");
    PJRT_Client* c = args->device->client;
    args->bytes_in_use = c ? c->live_buffer_bytes.load() : 0;
    args->peak_bytes_in_use = c ? c->peak_buffer_bytes.load() : 0;
    args->peak_bytes_in_use_is_set = c != nullptr;
    args->num_allocs = c ? c->num_allocs.load() : 0;
    args->num_allocs_is_set = c != nullptr;
    args->largest_alloc_size_is_set = false;
    args->bytes_limit_is_set = false;
    args->bytes_reserved_is_set = false;
    args->peak_bytes_reserved_is_set = false;
    args->bytes_reservable_limit_is_set = false;
    args->largest_free_block_bytes_is_set = false;
    args->pool_bytes_is_set = false;
    args->peak_pool_bytes_is_set = false;
    return nullptr;
}

// ---- memories (PJRTMemory.swift:60-136) ----
PJRT_Error* memory_id(PJRT_Memory_Id_Args* args) {
    PJRT_B200_REQUIRE(args && args->memory, "NULL args");
    args->id = args->memory->id;
    return nullptr;
}
PJRT_Error* memory_kind(PJRT_Memory_Kind_Args* args) {
    PJRT_B200_REQUIRE(args && args->memory, "NULL args");
    args->kind = args->memory->kind.c_str();
    args->kind_size = args->memory->kind.size();
    return nullptr;
}
PJRT_Error* memory_kind_id(PJRT_Memory_Kind_Id_Args* args) {
    PJRT_B200_REQUIRE(args && args->memory, "NULL args");
    args->kind_id = args->memory->kind_id;
    return nullptr;
}
PJRT_Error* memory_debug_string(PJRT_Memory_DebugString_Args* args) {
    PJRT_B200_REQUIRE(args && args->memory, "NULL args");
    args->debug_string = args->memory->debug_string.c_str();
    args->debug_string_size = args->memory->debug_string.size();
    return nullptr;
}
PJRT_Error* memory_to_string(PJRT_Memory_ToString_Args* args) {
    PJRT_B200_REQUIRE(args && args->memory, "NULL args");
    args->to_string = args->memory->to_string.c_str();
    args->to_string_size = args->memory->to_string.size();
    return nullptr;
}
PJRT_Error* memory_addressable_by_devices(PJRT_Memory_AddressableByDevices_Args* args) {
    PJRT_B200_REQUIRE(args && args->memory, "NULL args");
    args->devices = args->memory->devices.data();
    args->num_devices = args->memory->devices.size();
    return nullptr;
}

// ---- topology (PJRTTopology.swift:40-104) ----
PJRT_Error* topology_platform_name(PJRT_TopologyDescription_PlatformName_Args* args) {
    PJRT_B200_REQUIRE(args, "NULL args");
    args->platform_name = kPlatformName;
    args->platform_name_size = sizeof(kPlatformName) - 1;
    return nullptr;
}
PJRT_Error* topology_platform_version(PJRT_TopologyDescription_PlatformVersion_Args* args) {
    PJRT_B200_REQUIRE(args, "NULL args");
    args->platform_version = kPlatformVersion;
    args->platform_version_size = sizeof(kPlatformVersion) - 1;
    return nullptr;
}
PJRT_Error* topology_device_descriptions(PJRT_TopologyDescription_GetDeviceDescriptions_Args* args) {
    PJRT_B200_REQUIRE(args && args->topology, "NULL args");
    args->descriptions = args->topology->descriptions.data();
    args->num_descriptions = args->topology->descriptions.size();
    return nullptr;
}
PJRT_Error* topology_serialize(PJRT_TopologyDescription_Serialize_Args*) {
    return make_error(PJRT_Error_Code_UNIMPLEMENTED, "TopologyDescription_Serialize not implemented");
}
PJRT_Error* topology_attributes(PJRT_TopologyDescription_Attributes_Args* args) {
    PJRT_B200_REQUIRE(args, "NULL args");
    args->attributes = nullptr;
    args->num_attributes = 0;
    return nullptr;
}

}  // namespace

void fill_client_api(PJRT_Api* api) {
    api->PJRT_Client_Create = client_create;
    api->PJRT_Client_Destroy = client_destroy;
    api->PJRT_Client_PlatformName = client_platform_name;
    api->PJRT_Client_ProcessIndex = client_process_index;
    api->PJRT_Client_PlatformVersion = client_platform_version;
    api->PJRT_Client_Devices = client_devices;
    api->PJRT_Client_AddressableDevices = client_addressable_devices;
    api->PJRT_Client_LookupDevice = client_lookup_device;
    api->PJRT_Client_LookupAddressableDevice = client_lookup_addressable_device;
    api->PJRT_Client_AddressableMemories = client_addressable_memories;
    api->PJRT_Client_DefaultDeviceAssignment = client_default_device_assignment;
    api->PJRT_Client_TopologyDescription = client_topology_description;
    api->PJRT_DeviceDescription_Id = dd_id;
    api->PJRT_DeviceDescription_ProcessIndex = dd_process_index;
    api->PJRT_DeviceDescription_Attributes = dd_attributes;
    api->PJRT_DeviceDescription_Kind = dd_kind;
    api->PJRT_DeviceDescription_DebugString = dd_debug_string;
    api->PJRT_DeviceDescription_ToString = dd_to_string;
    api->PJRT_Device_GetDescription = device_get_description;
    api->PJRT_Device_IsAddressable = device_is_addressable;
    api->PJRT_Device_LocalHardwareId = device_local_hardware_id;
    api->PJRT_Device_AddressableMemories = device_addressable_memories;
    api->PJRT_Device_DefaultMemory = device_default_memory;
    api->PJRT_Device_MemoryStats = device_memory_stats;
    api->PJRT_Memory_Id = memory_id;
    api->PJRT_Memory_Kind = memory_kind;
    api->PJRT_Memory_Kind_Id = memory_kind_id;
    api->PJRT_Memory_DebugString = memory_debug_string;
    api->PJRT_Memory_ToString = memory_to_string;
    api->PJRT_Memory_AddressableByDevices = memory_addressable_by_devices;
    api->PJRT_TopologyDescription_PlatformName = topology_platform_name;
    api->PJRT_TopologyDescription_PlatformVersion = topology_platform_version;
    api->PJRT_TopologyDescription_GetDeviceDescriptions = topology_device_descriptions;
    api->PJRT_TopologyDescription_Serialize = topology_serialize;
    api->PJRT_TopologyDescription_Attributes = topology_attributes;
}

}  // namespace pjrt_b200
