// Compiler-core interfaces: pass pipeline, static memory plan and the compiled executable.
// The reference counterparts are MetalHLOCompiler (Sources/MetalHLOCore/Compiler/MetalHLOCompiler.swift:154-252),
// PassManager (Compiler/PassManager.swift), StaticMemoryPlanner (Memory/StaticMemoryPlanner.swift) and
// IntegratedExecutor (Runtime/IntegratedExecutor.swift).
#pragma once

#include <functional>
#include <memory>
#include <set>
#include <string>
#include <vector>

#include "ir.h"

namespace mhlo {

// How a function is split over `count` equal, contiguous shards of its batch; this compilation builds shard `index`.
struct ShardSpec {
    int count = 1, index = 0;
    std::vector<int> input_axes;  // per argument: the split axis, -1 = replicated. Empty = chosen by shard_function.
};
// What shard_function decided: the split axis of every argument and result (-1 = replicated, the same on every shard)
// and their types before the split.
struct ShardPlan {
    int count = 1, index = 0;
    std::vector<int> input_axes, output_axes;
    std::vector<TensorType> full_input_types, full_output_types;
};

struct CompileOptions {
    ShardSpec shard;             // count > 1: compile one shard of the batch (shard.cpp)
    int opt_level = 2;           // 0..3, same meaning as MHLOOptimizationLevel
    bool enable_caching = true;
    bool enable_debug_info = false;
    bool has_enabled_set = false;
    std::set<std::string> enabled_passes;   // when has_enabled_set: only these run
    std::set<std::string> disabled_passes;  // never run (METALHLO_DISABLED_PASSES)
};

struct PassRecord {
    std::string name;
    bool ran = false;
    bool changed = false;
    int ops_before = 0, ops_after = 0;
};

// Names of every registered pass in pipeline order (Compiler/PassManager.swift:121-237).
const std::vector<std::string>& all_pass_names();
// The pass set an optimisation level enables (Sources/MetalHLO/CompilationConfig.swift:232-263).
std::set<std::string> passes_for_level(int opt_level);
// Runs the pipeline once over f (single sweep, as the reference does). Returns one record per registered pass.
std::vector<PassRecord> run_pass_pipeline(Function& f, const CompileOptions& options);

// ---- flattening (inline.cpp) ----
// Inlines every `call` of @main (transitively) from the module's other functions. True when something changed.
bool inline_calls(Module& m);
// Unrolls stablehlo.while loops whose trip count is static: a counter compared with a constant in the condition,
// advanced by a constant in the body, starting from a constant. Other loops are left in place.
bool unroll_static_whiles(Function& f);
// Replaces stablehlo.if / stablehlo.case by their branches, all computed, and `select`s on the selector.
bool flatten_conditionals(Function& f);
// Replaces stablehlo.map by its computation applied to whole tensors.
bool flatten_maps(Function& f);
// Runs the pass pipeline on the bodies of the loops that stay loops (after it ran on the function itself).
void optimize_loop_bodies(Function& f, const CompileOptions& options);
// Replaces chlo.top_k by iota + stable descending sort + slices.
bool flatten_top_k(Function& f);
// Replaces the results of stablehlo.optimization_barrier by its operands.
bool drop_optimization_barriers(Function& f);
// All four, repeated until none applies; returns the flattened @main.
Function flatten_main(Module& m);

// ---- MLIR bytecode (bytecode.cpp) ----
bool is_mlir_bytecode(const char* data, size_t size);
// Converts an MLIR bytecode program to StableHLO text by running the jaxlib helper script in a child process
// (METALHLO_PYTHON, METALHLO_BYTECODE_HELPER, METALHLO_HELPER_TIMEOUT_S). False with a message in *why otherwise.
bool bytecode_to_text(const char* bytecode, size_t size, std::string* text, std::string* why);

// ---- batch sharding (shard.cpp) ----
// Proves that every result of f is either the same on every shard or, slice by slice along one axis, a function of the
// same slice of the split arguments, and rewrites f to compute shard spec.index of spec.count. Throws
// CompileError(4, ...) naming the operator that mixes elements along the split axis when no such proof exists.
ShardPlan shard_function(Function& f, const ShardSpec& spec);

// ---- memory plan -----------------------------------------------------------------------------------------------

struct PlanInterval {
    int64_t bytes = 0;
    int first = 0, last = 0;  // inclusive step range in which the buffer is live
    int64_t offset = -1;      // assigned by plan_memory
};
// Lifetime-interval offset assignment into one arena: largest buffers first, each at the lowest 256-byte
// aligned offset that does not overlap a buffer whose lifetime intersects; total rounded up to 4096
// (Memory/StaticMemoryPlanner.swift:175-253,486-554). Returns the arena size.
int64_t plan_memory(std::vector<PlanInterval>* buffers);

// ---- executable ------------------------------------------------------------------------------------------------

struct ExecutionStats {
    int64_t count = 0;
    double total_ms = 0, last_ms = 0;
};

class Executable {
  public:
    ~Executable();
    // Parses, optimises, lowers and plans `mlir`; uploads constants and allocates the arena on the current CUDA
    // device. Throws CompileError.
    static std::unique_ptr<Executable> compile(const std::string& mlir, const CompileOptions& options);
    // The same without touching a device: the step list, launch count and memory plan of `mlir`. The result cannot run.
    static std::unique_ptr<Executable> plan_only(const std::string& mlir, const CompileOptions& options);

    int num_inputs() const { return static_cast<int>(input_types_.size()); }
    int num_outputs() const { return static_cast<int>(output_types_.size()); }
    const TensorType& input_type(int i) const { return input_types_[i]; }
    const TensorType& output_type(int i) const { return output_types_[i]; }

    // Enqueues the whole program on `stream`. inputs/outputs are device pointers to dense row-major tensors of the
    // declared types. Returns 0 or an MHLO status code (message via last_error()).
    int execute(const void* const* inputs, void* const* outputs, void* stream);
    const std::string& last_error() const { return error_; }

    int num_steps() const { return static_cast<int>(steps_.size()); }
    int num_kernel_launches() const { return launches_per_run_; }
    int64_t arena_bytes() const { return arena_bytes_; }
    int64_t constant_bytes() const { return static_cast<int64_t>(const_pool_.size()); }
    const std::vector<PassRecord>& pass_log() const { return pass_log_; }
    const std::string& optimized_text() const { return optimized_text_; }
    const ShardPlan& shard_plan() const { return shard_plan_; }
    const std::vector<PlanInterval>& plan_intervals() const { return plan_intervals_; }  // the arena buffers as planned
    std::vector<std::string> step_labels() const;
    ExecutionStats stats;

  private:
    friend class Lowering;
    struct Ctx {
        const void* const* inputs;
        void* const* outputs;
        char* arena;
        char* consts;
        void* stream;
    };
    struct Step {
        std::string label;
        std::string detail;  // result type of the op the step was lowered from (shown by the per-step profile)
        int launches = 1;
        std::function<int(const Ctx&)> run;  // returns an mhlo_cuda status
    };
    std::vector<TensorType> input_types_, output_types_;
    std::vector<Step> steps_;
    std::vector<uint8_t> const_pool_;
    char* const_dev_ = nullptr;
    char* arena_dev_ = nullptr;
    int64_t arena_bytes_ = 0;
    int launches_per_run_ = 0;
    std::vector<PassRecord> pass_log_;
    std::string optimized_text_;
    ShardPlan shard_plan_;
    std::vector<PlanInterval> plan_intervals_;
    std::string error_;

    // CUDA-graph replay of the launch list. A (stream, input pointers, output pointers) combination that comes back
    // is recorded once and replayed from then on; combinations seen once run launch by launch.
    struct GraphSlot {
        std::vector<const void*> key;  // stream, inputs..., outputs...
        void* graph = nullptr;         // instantiated graph; null until the key has been seen twice
        uint64_t last_use = 0;
    };
    std::vector<GraphSlot> graph_slots_;
    uint64_t graph_clock_ = 0;
    bool graphs_usable_ = true;  // cleared when a capture of this program failed
    bool host_control_ = false;  // the program has a loop that the host drives: it synchronises, so it is never recorded
    int run_steps(const Ctx& c, bool debug, bool profile);
  public:
    int64_t graph_replays = 0;   // executions served by a graph launch
};

// Small helpers over backend_config JSON strings of fused custom calls.
double json_number(const std::string& json, const std::string& key, double dflt);
bool json_bool(const std::string& json, const std::string& key, bool dflt);
std::string json_string(const std::string& json, const std::string& key, const std::string& dflt);
std::vector<int64_t> json_int_array(const std::string& json, const std::string& key);

}  // namespace mhlo
