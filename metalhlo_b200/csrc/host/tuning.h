// Kernel tuning: a persistent database of measured launch configurations and the tuner that fills it.
// Counterpart of TuningDatabase (Sources/MetalHLOCore/Tuning/TuningDatabase.swift:15-290) and AutoTuner
// (Tuning/AutoTuner.swift:108-764): same key (operation, shapes, dtype, device name), same record (best configuration,
// median time, GFLOP/s, candidates tried, timestamp), same measurement protocol (5 warm-up + 20 timed runs, median),
// same JSON layout (version, entries as alternating key/value array, savedAt). The configuration carries this
// backend's knobs instead of Metal's simdgroup tiles.
#pragma once

#include <cstdint>
#include <map>
#include <mutex>
#include <string>
#include <vector>

namespace mhlo {

struct TuningKey {
    std::string op_type;  // "fused_layer_norm", "fused_rms_norm", "fused_softmax", "dot_general"
    std::vector<std::vector<int64_t>> shapes;
    std::string dtype;    // "bf16", "f16", "f32"
    std::string device;   // CUDA device name
    bool operator<(const TuningKey& o) const;
    bool operator==(const TuningKey& o) const;
};

// Launch knobs. Row kernels use threads / vectors_per_thread / ctas_per_sm (mhlo_cuda_row_tuning); the tile fields
// describe GEMM-shaped kernels (CTA tile and TMA pipeline depth). Zero = "library default".
struct TuningConfig {
    int32_t tile_m = 0, tile_n = 0, tile_k = 0, stages = 0;
    int32_t threads = 0, vectors_per_thread = 0, ctas_per_sm = 0;
    int32_t cta_group = 0;   // GEMM: 1 = one CTA per tile, 2 = a pair of CTAs per 256 x 256 tile (mhlo_cuda_gemm_tuning)
    int32_t tile_order = 0;  // attention: order of the query tiles over the CTAs (mhlo_cuda_attention_tuning)
    bool is_default() const {
        return !tile_m && !tile_n && !tile_k && !stages && !threads && !vectors_per_thread && !ctas_per_sm && !cta_group && !tile_order;
    }
    std::string description() const;
};

struct TuningRecord {
    TuningConfig best;
    double measured_time_s = 0;  // median of the timed runs
    double gflops = 0;           // 0 for bandwidth-bound kernels; gbytes_per_s is set instead
    double gbytes_per_s = 0;
    int32_t configs_tried = 0;
    double timestamp = 0;        // seconds since the Unix epoch
};

class TuningDatabase {
  public:
    // Loads `path` when it exists (a malformed file is ignored with a warning, as the reference does).
    explicit TuningDatabase(std::string path);
    bool get(const TuningKey& key, TuningRecord* out) const;
    void store(const TuningKey& key, const TuningRecord& record);
    bool remove(const TuningKey& key);
    void clear();
    size_t count() const;
    std::vector<TuningKey> keys() const;
    // Writes the file when something changed since the last save. False on an I/O error.
    bool save();
    // Merges the entries of another database file; existing keys win unless overwrite. Returns entries taken.
    int import_from(const std::string& other_path, bool overwrite);
    // Drops entries older than max_age_days; returns how many.
    int prune(double max_age_days, double now_epoch_s);
    std::string to_json() const;
    // Replaces the contents with those of a database document.
    bool from_json(const std::string& text, std::string* why);
    // Merges a database document (the file format); existing keys win unless overwrite. Returns entries taken, -1 on
    // a malformed document.
    int merge_json(const std::string& text, bool overwrite, std::string* why);
    const std::string& path() const { return path_; }

    // The process-wide database: the one open_global installed, else $METALHLO_TUNING_DB when set, else none
    // (nullptr = heuristics only).
    static TuningDatabase* global();
    // Installs (and loads) `path` as the process-wide database; an earlier one is saved first and stays allocated
    // because compiled executables may still be reading it.
    static TuningDatabase* open_global(const std::string& path);

  private:
    std::string path_;
    mutable std::mutex mu_;
    std::map<TuningKey, TuningRecord> entries_;
    bool dirty_ = false;
};

// Row-kernel candidates that are valid for `hidden` elements of `elem_bytes` (a thread holds vectors of 16 bytes).
std::vector<TuningConfig> row_kernel_candidates(int64_t hidden, int elem_bytes);

// Times every candidate of a row kernel on the current device (5 warm-up + 20 timed launches each, median, CUDA events)
// and returns the best; stores it in `db` when db is not null. kind: "fused_layer_norm" | "fused_rms_norm" |
// "fused_softmax". Scratch tensors are allocated and freed inside. Returns an mhlo_cuda status; message via *why.
int tune_row_kernel(const std::string& kind, int dtype, int64_t rows, int64_t hidden, int max_trials, TuningDatabase* db,
                    TuningRecord* out, std::string* why);

// Candidates of the tensor-core GEMM: tile width x ring depth x CTA group, as the kernel provides them.
std::vector<TuningConfig> gemm_candidates(int64_t m, int64_t n, int64_t k);

// Description of one dot_general as the tuner and the lowering key it: bf16 / f16 operands, `batch` independent products,
// operand majors as the kernel sees them (k_major: the contracted dimension is the contiguous one).
struct GemmCase {
    int dtype = 0, out_dtype = 0;
    int64_t batch = 1, m = 0, n = 0, k = 0;
    bool a_k_major = true, b_k_major = false;
    TuningKey key(const std::string& device) const;
};
// Times every candidate on the current device (5 warm-up + 20 timed launches, median) and stores the best under the
// case's key. Scratch operands are allocated and freed inside.
int tune_gemm(const GemmCase& c, int max_trials, TuningDatabase* db, TuningRecord* out, std::string* why);

struct AttentionCase {
    int dtype = 0;
    int64_t batch = 1, heads = 1, seq_q = 0, seq_k = 0, head_dim = 0;
    bool causal = false;
    bool bshd = false;  // operands laid out [batch, sequence, head, dim] instead of [batch, head, sequence, dim]
    TuningKey key(const std::string& device) const;
};
int tune_attention(const AttentionCase& c, int max_trials, TuningDatabase* db, TuningRecord* out, std::string* why);

// Name of the current CUDA device, as the keys carry it.
std::string current_device_name();

}  // namespace mhlo
