// nnabla extension backend "b200": backend singleton, device memory, array
// classes and registration entry point. Mirrors what the reference's own CPU
// backend provides (include/nbla/cpu.hpp, include/nbla/memory/cpu_memory.hpp,
// include/nbla/array/cpu_array.hpp, src/nbla/init.cpp.tmpl:44-111) for a CUDA
// device driven through the C ABI of libnnabla_b200.so.
#ifndef NBLA_B200_B200_HPP_
#define NBLA_B200_B200_HPP_

#include <nbla/array.hpp>
#include <nbla/backend_base.hpp>
#include <nbla/context.hpp>
#include <nbla/memory/allocator.hpp>
#include <nbla/memory/memory.hpp>
#include <nbla/singleton_manager.hpp>
#include <nbla/variable.hpp>

#include <string>
#include <vector>

namespace nbla {

using std::string;
using std::vector;

/** Registers the backend, its array classes, synchronizers and functions
    under "b200:float". Idempotent and thread-safe, like init_cpu(). */
void init_b200();

/** Context of this backend: Context({"b200:float"}, "B200CachedArray", device_id).
    There is no "cpu:float" entry: no function falls back to the CPU. */
Context b200_context(const string &device_id = "0", const string &type_config = "float");

/** Raises nbla::Exception for a non-zero status of the C ABI (the message is
    nb200_last_error()). */
void nb200_check(int status, const char *what);

/** Makes the context's device current and returns the stream every function,
    copy and fill of this backend is enqueued on for that device: one
    non-blocking stream per device, created at first use, never the legacy
    default stream. It is shared by the host threads that use the device on
    purpose: the caching allocator is shared by them too and hands a block that
    one thread released to the next thread that asks, with no record of the
    work still queued on it, so that work and the new owner's must be ordered
    by one stream. */
void *b200_stream(const string &device_id);

/** Bucket plan of the communicator's packed all-reduce: consecutive arrays (sizes in elements) are
    grouped into buckets of at most pack_size elements, a larger array alone; returns the index of
    the first array of every bucket, then the end index (ext/src/b200_communicator.cpp). */
vector<size_t> b200_plan_buckets(const vector<size_t> &sizes, size_t pack_size);

/** Counters of the paths the functions took since the last reset, by name:
    "int8_convolutions", "bf16_convolutions", "int8_affines",
    "weight_cache_hits", "weight_cache_misses". Unknown names read 0. */
long long b200_counter(const string &name);
void b200_count(const char *name);
void b200_reset_counters();

/** Device memory block (cudaMalloc through nb200_malloc). Same contract as
    CpuMemory (src/nbla/memory/cpu_memory.cpp:31-80). */
class B200Memory : public Memory {
public:
  B200Memory(size_t bytes, const string &device_id);
  B200Memory(size_t bytes, const string &device_id, void *ptr);
  ~B200Memory();

protected:
  bool alloc_impl() override;
  shared_ptr<Memory> divide_impl(size_t second_start) override;
  void merge_next_impl(Memory *from) override;
  void merge_prev_impl(Memory *from) override;
};

/** Backend singleton: array class list and the two allocators. */
class B200 : public BackendBase {
public:
  ~B200();
  vector<string> array_classes() const override;
  void _set_array_classes(const vector<string> &a) override;
  void register_array_class(const string &name) override;
  shared_ptr<Allocator> caching_allocator() override;
  shared_ptr<Allocator> naive_allocator() override;
  void free_unused_host_caches() override;
  void device_synchronize(const string &device) override;
  void default_stream_synchronize(const string &device) override;
  void create_lms_streams(int device = -1) override;

private:
  friend SingletonManager;
  B200();
};

/** Device array allocated from the backend's naive allocator. */
class B200Array : public Array {
public:
  explicit B200Array(const Size_t size, dtypes dtype, const Context &ctx, const AllocatorMemoryPtr mem = nullptr,
                     const Size_t offset = 0);
  virtual ~B200Array();
  virtual void copy_from(const Array *src_array);
  virtual void zero();
  virtual void fill(float value);
  static Context filter_context(const Context &ctx);
};

/** Device array allocated from the backend's caching allocator. */
class B200CachedArray : public B200Array {
public:
  explicit B200CachedArray(const Size_t size, dtypes dtype, const Context &ctx,
                           const AllocatorMemoryPtr mem = nullptr, const Size_t offset = 0);
  virtual ~B200CachedArray();
  static Context filter_context(const Context &ctx);
};

/** Identity of the current contents of a variable's data. Two equal, valid
    stamps mean nothing wrote to the array in between.

    SyncedArray::modification_count (include/nbla/synced_array.hpp:183) cannot
    serve alone: every cast() runs clear_all_array(), which sets the count to 0,
    and then increments it (src/nbla/synced_array.cpp:185-193, :484-489), so it
    reads 1 after every write; only zero() and fill() move it further. The
    stamp therefore also carries a write generation that this backend keeps
    itself through nnabla's SyncedArrayCallback hook (synced_array.hpp:310-345):
    every CAST or CLEAR of any SyncedArray, on any backend, gives that array a
    new, never repeated generation. The hook is a single process-wide slot; if
    another component takes it over (the LMS scheduler does), generations stop
    moving, so write_tracking_alive() probes the hook and stamps taken while it
    is dead are invalid (valid == false, never equal to anything). */
struct DataStamp {
  const SyncedArray *array = nullptr;
  size_t count = 0;
  unsigned long long generation = 0;
  bool valid = false;
  bool operator==(const DataStamp &o) const {
    return valid && o.valid && array == o.array && count == o.count && generation == o.generation;
  }
  bool operator!=(const DataStamp &o) const { return !(*this == o); }
};
DataStamp data_stamp(const Variable *v);
bool write_tracking_alive();

/** Fixed-point tags: which arrays currently hold the output of
    FixedPointQuantize with at most 8 bits, and with which step size. The
    contraction functions consult them to take the exact int8 tensor-core path.
    A tag is the data stamp at the time of tagging: any later write to the array
    (by any backend) makes it stale. */
void fxp_tag_set(const Variable *v, float delta);
float fxp_tag_get(const Variable *v); // 0 when untagged or stale
/** The same tag with the int8 channel-last codes of the tensor (nb200_fixed_point_quantize_nhwc_codes_f32),
    which the quantizer wrote in the pass that made it; a convolution that finds them does not convert the
    fp32 values again. The codes live as long as the tag (until the array is written or tagged again). */
void fxp_tag_set(const Variable *v, float delta, const NdArrayPtr &codes);
NdArrayPtr fxp_tag_codes(const Variable *v); // nullptr when untagged, stale or tagged without codes

} // namespace nbla
#endif
