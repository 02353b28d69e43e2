// The seam between the engine (scheduler, paged block pool, state slots, step packing, sampling, C ABI) and a model design
// that is not the built-in Llama kernel sequence.  The engine owns sequences, pages and slots; a Model owns its weights,
// its per-layer caches / recurrent states (sized from the pool the engine hands it) and turns one packed step into logits
// and sampled ids.  Designs register by the "architecture" string of their config.json (model_registry.cc).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include <memory>
#include <string>
#include <unordered_map>
#include <vector>

#include "../../include/b200engine.h"
#include "hostutil.h"
#include "mixers.h"

namespace b200 {

// One scheduler step as the kernels see it (device pointers into the step's packed input buffer).
struct StepBatch {
  int T = 0;        // tokens in the step
  int nseq = 0;     // sequences in the step
  int S = 0;        // rows whose logits are wanted
  const int* ids = nullptr;         // [T]
  const int* prev_ids = nullptr;    // [T] the token before each token in its sequence, -1 at position 0
  const int* pos = nullptr;         // [T]
  const int* slots = nullptr;       // [T] page * page_size + offset of each token's cache row
  const int* rows = nullptr;        // [S] token rows whose logits are wanted
  const int* seq_of_tok = nullptr;  // [T] index of the token's sequence within the step
  const int* seqs = nullptr;        // [nseq][8] = {first row, rows, first position, state slot, 0, 0, 0, 0}
  const int* btab = nullptr;        // [nseq][max_blocks]
  int max_blocks = 0;
  int max_ctx = 0;                  // longest context in the step: max over sequences of first position + rows
};

struct ModelEnv {
  cudaStream_t stream;
  int device, sms;
  int Tcap;              // most tokens in a step
  int max_model_len;
  int page;              // tokens per page of the block pool
  int64_t num_blocks;    // pages in the pool
  int num_slots;         // recurrent-state slots (one per live sequence)
};

struct TensorRef {
  void* ptr;
  size_t bytes;
};

class CheckpointReader;   // loader.cc

class Model {
 public:
  virtual ~Model() {}
  virtual const char* arch() const = 0;
  virtual int vocab() const = 0;
  virtual size_t cache_bytes_per_block(int page) const = 0;   // over all layers that cache per token
  virtual size_t state_bytes_per_slot() const = 0;            // over all recurrent layers (0: no slots needed)
  // the most tokens back any caching layer looks (itself included); 0 = some layer sees the whole sequence.  The engine
  // returns pages that lie wholly before every such window to the pool while the sequence is still running.
  virtual int cache_window() const { return 0; }
  // the first tokens of a sequence that stay visible to every later token whatever the window: their pages are not returned
  virtual int cache_keep_first() const { return 0; }
  // the most positions a sequence may have (a learned position table has that many rows); 0 = no limit of the design's own.
  // The engine lowers its max_model_len to it.
  virtual int max_positions() const { return 0; }
  // allocate weights (unset), activations for env.Tcap tokens, caches for env.num_blocks pages, states for env.num_slots
  virtual int init(const ModelEnv& env) = 0;
  // sizes that only the checkpoint's tensor shapes give; called before init() when there is a checkpoint
  virtual int inspect(const CheckpointReader& ck, std::string* err) { return 0; }
  virtual int load(const CheckpointReader& ck, std::string* err) = 0;
  virtual int randomize(uint64_t seed) = 0;
  // Run the step.  sampled [S] (device) gets the argmax of every wanted row; host_logits (optional, pinned or pageable
  // host memory, [S, vocab] fp32) gets the logits themselves (copies are enqueued on the stream).  *launches += kernels.
  virtual int forward(const StepBatch& b, int* sampled, float* host_logits, int64_t* launches) = 0;
  // debug: when set, forward() appends the fp32 residual [T, width] after every layer run (synchronising)
  std::vector<float>* residual_sink = nullptr;
  // debug: per-kernel device time; when on, forward() waits for every launch (name -> (microseconds, launches))
  bool profile_kernels = false;
  std::unordered_map<std::string, std::pair<double, int64_t>> kernel_times;
  std::unordered_map<std::string, TensorRef> tensors;   // named device tensors (weights), for inspection
};

typedef std::unique_ptr<Model> (*ModelFactory)(const JVal& config, DType dtype, std::string* err);
// nullptr when no design registered that architecture string
ModelFactory find_model_factory(const std::string& arch);
std::string registered_architectures();

// loader.cc: read access to a safetensors checkpoint (directory, shard index or single file)
class CheckpointReader {
 public:
  CheckpointReader();
  ~CheckpointReader();
  bool open(const std::string& path, std::string* err);
  bool has(const std::string& name) const;
  bool shape(const std::string& name, std::vector<int64_t>* out) const;
  // the tensor as fp32 (BF16 / F16 / F32 / I32 sources), with its shape
  bool read_f32(const std::string& name, std::vector<float>* out, std::vector<int64_t>* shape, std::string* err) const;
 private:
  struct Impl;
  Impl* impl_;
};

}  // namespace b200

namespace b200 {
// engine.cu: an engine whose forward pass is `mdl` (weights unset: load or randomize through engine_model)
int engine_create_with_model(const b200_config* cfg, std::unique_ptr<Model> mdl, b200_engine** out);
Model* engine_model(b200_engine* e);

std::unique_ptr<Model> make_nomanex(const JVal& config, DType dtype, std::string* err);
std::unique_ptr<Model> make_zinavik(const JVal& config, DType dtype, std::string* err);
std::unique_ptr<Model> make_mulenex(const JVal& config, DType dtype, std::string* err);
std::unique_ptr<Model> make_nagilix(const JVal& config, DType dtype, std::string* err);

}  // namespace b200
