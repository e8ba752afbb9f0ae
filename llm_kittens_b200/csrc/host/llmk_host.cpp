// Host runtime of the framework (no CUDA): random numbers, token-shard data loader, multiple-choice
// eval loader and tokenizer, exported with a C ABI for ctypes.
//
// File formats are those of the reference (llmc/dataloader.h:27-31, 330-348; llmc/tokenizer.h:25-105)
// so that existing .bin shards, eval files and tokenizer files load unchanged, and the shuffling
// random stream is the same (MT19937 seeded with 42 + rank, Fisher-Yates with `rand % (i+1)`), so a
// loader position saved by one implementation can be resumed by the other. The implementation is
// different: shards are memory-mapped and a batch is widened straight from the mapping into the
// caller's (pinned) int32 buffers, there are no process-wide exits (errors are returned as codes and
// a message), and all state lives in C++ objects behind opaque handles.
#include <fcntl.h>
#include <glob.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <algorithm>
#include <cmath>
#include <string>
#include <vector>

#define HOST_API extern "C" __attribute__((visibility("default")))

namespace {

thread_local std::string g_error;
int fail(const std::string& msg) {
    g_error = msg;
    return -1;
}

// ------------------------------------------------------------------------------------------ MT19937
// Standard Mersenne Twister (Matsumoto & Nishimura) with the output conventions of PyTorch's CPU
// generator, so `normal`/`uniform`/permutations reproduce torch.manual_seed(seed) streams.
class Mt19937 {
public:
    static constexpr int N = 624, M = 397;
    explicit Mt19937(uint32_t seed = 5489u) { reseed(seed); }
    void reseed(uint32_t seed) {
        seed_ = seed;
        mt_[0] = seed;
        for (int i = 1; i < N; i++) mt_[i] = 1812433253u * (mt_[i - 1] ^ (mt_[i - 1] >> 30)) + (uint32_t)i;
        left_ = 1;
        next_ = 0;
    }
    uint32_t next_u32() {
        if (--left_ <= 0) twist();
        uint32_t y = mt_[next_++];
        y ^= y >> 11;
        y ^= (y << 7) & 0x9d2c5680u;
        y ^= (y << 15) & 0xefc60000u;
        y ^= y >> 18;
        return y;
    }
    uint64_t next_u64() {
        const uint64_t hi = next_u32();
        return (hi << 32) | next_u32();
    }
    float next_f32() { return (float)(next_u32() & ((1u << 24) - 1)) * (1.0f / (float)(1u << 24)); }
    double next_f64() { return (double)(next_u64() & ((1ull << 53) - 1)) * (1.0 / (double)(1ull << 53)); }

    // serialised layout (2520 bytes): u64 seed, i32 left, u32 next, u32 state[624], u32 {0, 0x9908b0df}
    static constexpr size_t kStateBytes = 8 + 4 + 4 + 4 * N + 8;
    void save(uint8_t* out) const {
        uint64_t s = seed_;
        memcpy(out, &s, 8);
        memcpy(out + 8, &left_, 4);
        memcpy(out + 12, &next_, 4);
        memcpy(out + 16, mt_, 4 * N);
        const uint32_t mag[2] = {0u, 0x9908b0dfu};
        memcpy(out + 16 + 4 * N, mag, 8);
    }
    void load(const uint8_t* in) {
        uint64_t s;
        memcpy(&s, in, 8);
        seed_ = s;
        memcpy(&left_, in + 8, 4);
        memcpy(&next_, in + 12, 4);
        memcpy(mt_, in + 16, 4 * N);
    }

private:
    void twist() {
        static const uint32_t mag[2] = {0u, 0x9908b0dfu};
        for (int k = 0; k < N; k++) {
            const uint32_t y = (mt_[k] & 0x80000000u) | (mt_[(k + 1) % N] & 0x7fffffffu);
            mt_[k] = mt_[(k + M) % N] ^ (y >> 1) ^ mag[y & 1u];
        }
        left_ = N;
        next_ = 0;
    }
    uint64_t seed_ = 0;
    int32_t left_ = 1;
    uint32_t next_ = 0;
    uint32_t mt_[N];
};

// torch.normal_ on CPU: tensors of >= 16 elements are filled with uniforms and transformed by
// Box-Muller in blocks of 16 (first 8 with cos, last 8 with sin), the ragged tail redoes the last 16.
void box_muller_16(float* d, float mean, float std) {
    for (int t = 0; t < 8; t++) {
        const float u1 = 1.0f - d[t];
        const float u2 = d[t + 8];
        const float radius = sqrtf(-2.0f * logf(u1 + 1e-12f));
        const float theta = (float)(2.0 * M_PI * u2);
        d[t] = radius * cosf(theta) * std + mean;
        d[t + 8] = radius * sinf(theta) * std + mean;
    }
}
void normal_fill(Mt19937& g, float* data, size_t n, float mean, float std) {
    if (n >= 16) {
        for (size_t i = 0; i < n; i++) data[i] = g.next_f32();
        for (size_t i = 0; i + 16 <= n; i += 16) box_muller_16(data + i, mean, std);
        if (n % 16 != 0) {
            float* tail = data + n - 16;
            for (int i = 0; i < 16; i++) tail[i] = g.next_f32();
            box_muller_16(tail, mean, std);
        }
        return;
    }
    bool have = false;
    double spare = 0.0;
    for (size_t i = 0; i < n; i++) {
        if (have) {
            data[i] = (float)(spare * std + mean);
            have = false;
            continue;
        }
        const float u1 = (float)g.next_f64();
        const float u2 = (float)g.next_f64();
        const float radius = sqrtf(-2.0f * logf(1.0f - u2 + 1e-12f));
        const float theta = (float)(2.0 * M_PI * u1);
        spare = radius * sinf(theta);
        have = true;
        data[i] = radius * cosf(theta) * std + mean;
    }
}
void shuffle_ints(Mt19937& g, int* data, int n) {
    for (int i = n - 1; i > 0; i--) {
        const int j = (int)(g.next_u32() % (uint32_t)(i + 1));
        std::swap(data[i], data[j]);
    }
}

// ------------------------------------------------------------------------------------------ mapped file
class MappedFile {
public:
    ~MappedFile() { close(); }
    int open(const std::string& path) {
        close();
        fd_ = ::open(path.c_str(), O_RDONLY);
        if (fd_ < 0) return fail("cannot open " + path);
        struct stat st;
        if (fstat(fd_, &st) != 0) return fail("cannot stat " + path);
        size_ = (size_t)st.st_size;
        if (size_ == 0) return fail("empty file " + path);
        base_ = (const uint8_t*)mmap(nullptr, size_, PROT_READ, MAP_PRIVATE, fd_, 0);
        if (base_ == MAP_FAILED) {
            base_ = nullptr;
            return fail("mmap failed for " + path);
        }
        madvise((void*)base_, size_, MADV_SEQUENTIAL);
        return 0;
    }
    void close() {
        if (base_) munmap((void*)base_, size_);
        if (fd_ >= 0) ::close(fd_);
        base_ = nullptr;
        fd_ = -1;
        size_ = 0;
    }
    const uint8_t* data() const { return base_; }
    size_t size() const { return size_; }

private:
    int fd_ = -1;
    const uint8_t* base_ = nullptr;
    size_t size_ = 0;
};

constexpr int kHeaderInts = 256;
constexpr size_t kHeaderBytes = kHeaderInts * sizeof(int32_t);

int token_bytes_for_train_magic(int magic, int version, const std::string& path) {
    if (magic == 20240520) return version == 1 ? 2 : fail("bad version in " + path + " (gpt-2 shards are version 1)");
    if (magic == 20240801) return version == 7 ? 4 : fail("bad version in " + path + " (llama-3 shards are version 7)");
    return fail("bad magic in data file " + path + ": expected 20240520 (uint16 tokens) or 20240801 (uint32 tokens)");
}

// ------------------------------------------------------------------------------------------ DataLoader
class DataLoader {
public:
    int init(const char* pattern, size_t B, size_t T, int rank, int nproc, int shuffle) {
        B_ = B; T_ = T; rank_ = rank; nproc_ = nproc; shuffle_ = shuffle != 0;
        glob_t gl;
        if (glob(pattern, 0, nullptr, &gl) != 0 || gl.gl_pathc == 0) {
            globfree(&gl);
            return fail(std::string("no files match the pattern: ") + pattern);
        }
        for (size_t i = 0; i < gl.gl_pathc; i++) paths_.push_back(gl.gl_pathv[i]);
        globfree(&gl);
        if (shuffle_) {
            rng_.reseed(42u + (uint32_t)rank);
            shard_order_.resize(paths_.size());
            for (size_t i = 0; i < paths_.size(); i++) shard_order_[i] = (int)i;
        }
        num_tokens_ = 0;
        for (size_t i = 0; i < paths_.size(); i++) {
            int64_t ntok = 0;
            if (probe(paths_[i], &ntok)) return -1;
            if (ntok < (int64_t)(nproc_ * B_ * T_ + 1)) return fail("shard " + paths_[i] + " holds fewer tokens than one global batch + 1");
            num_tokens_ += (size_t)ntok;
        }
        return reset();
    }
    int reset() {
        shard_idx_ = 0;
        sample_idx_ = 0;
        if (shuffle_) shuffle_ints(rng_, shard_order_.data(), (int)shard_order_.size());
        if (load_shard((int)shard_idx_)) return -1;
        if (shuffle_) make_sample_order();
        return 0;
    }
    int next(int32_t* inputs, int32_t* targets) {
        if (sample_idx_ >= shard_samples_) {
            if (advance()) return -1;
        }
        const size_t idx = shuffle_ ? (size_t)sample_order_[sample_idx_] : sample_idx_;
        const size_t global_bytes = nproc_ * B_ * T_ * (size_t)token_bytes_;
        const size_t off = kHeaderBytes + idx * global_bytes + (size_t)rank_ * B_ * T_ * token_bytes_;
        const size_t n = B_ * T_;
        if (off + (n + 1) * token_bytes_ > file_.size()) return fail("batch runs past the end of " + paths_[current_path_]);
        if (token_bytes_ == 2) {
            const uint16_t* src = (const uint16_t*)(file_.data() + off);
            for (size_t i = 0; i < n; i++) {
                inputs[i] = src[i];
                targets[i] = src[i + 1];
            }
        } else {
            const uint32_t* src = (const uint32_t*)(file_.data() + off);
            for (size_t i = 0; i < n; i++) {
                if (src[i] > 0x7fffffffu || src[i + 1] > 0x7fffffffu) return fail("token id does not fit in int32");
                inputs[i] = (int32_t)src[i];
                targets[i] = (int32_t)src[i + 1];
            }
        }
        sample_idx_ += 1;
        return 0;
    }
    int resume(size_t shard_idx, size_t sample_idx) {
        shard_idx_ = shard_idx;
        sample_idx_ = sample_idx;
        return load_shard((int)shard_idx_);
    }
    // shuffle state blob: u64 n_shards, i32 shard_order[n], u64 n_samples, i32 sample_order[m], MT19937 state
    size_t shuffle_state_bytes() const {
        return shuffle_ ? 8 + 4 * shard_order_.size() + 8 + 4 * sample_order_.size() + Mt19937::kStateBytes : 0;
    }
    void save_shuffle_state(uint8_t* out) const {
        uint64_t n = shard_order_.size();
        memcpy(out, &n, 8); out += 8;
        memcpy(out, shard_order_.data(), 4 * n); out += 4 * n;
        uint64_t m = sample_order_.size();
        memcpy(out, &m, 8); out += 8;
        memcpy(out, sample_order_.data(), 4 * m); out += 4 * m;
        rng_.save(out);
    }
    int load_shuffle_state(const uint8_t* in, size_t nbytes) {
        if (!shuffle_) return fail("loader was not created with shuffling");
        const uint8_t* end = in + nbytes;
        uint64_t n, m;
        if (in + 8 > end) return fail("truncated shuffle state");
        memcpy(&n, in, 8); in += 8;
        if (n != paths_.size() || in + 4 * n + 8 > end) return fail("shuffle state does not match the shard list");
        shard_order_.resize(n);
        memcpy(shard_order_.data(), in, 4 * n); in += 4 * n;
        memcpy(&m, in, 8); in += 8;
        if (in + 4 * m + Mt19937::kStateBytes > end) return fail("truncated shuffle state");
        sample_order_.resize(m);
        memcpy(sample_order_.data(), in, 4 * m); in += 4 * m;
        rng_.load(in);
        return 0;
    }
    size_t B_ = 0, T_ = 0, num_tokens_ = 0, shard_samples_ = 0, shard_idx_ = 0, sample_idx_ = 0;
    int token_bytes_ = 0, magic_ = 0;
    std::vector<std::string> paths_;

private:
    int probe(const std::string& path, int64_t* ntok) {
        FILE* f = fopen(path.c_str(), "rb");
        if (!f) return fail("cannot open " + path);
        int32_t hdr[kHeaderInts];
        const size_t got = fread(hdr, sizeof(int32_t), kHeaderInts, f);
        fseek(f, 0, SEEK_END);
        const int64_t size = ftell(f);
        fclose(f);
        if (got != (size_t)kHeaderInts) return fail("short header in " + path);
        const int tb = token_bytes_for_train_magic(hdr[0], hdr[1], path);
        if (tb < 0) return -1;
        if (token_bytes_ == 0) {
            token_bytes_ = tb;
            magic_ = hdr[0];
        } else if (token_bytes_ != tb || magic_ != hdr[0]) {
            return fail("mixed data shard formats are not supported (" + path + ")");
        }
        *ntok = hdr[2];
        if (*ntok <= 0) return fail("no tokens in " + path);
        if (size != (int64_t)kHeaderBytes + *ntok * tb) return fail("file size of " + path + " does not match its header");
        return 0;
    }
    int load_shard(int order_idx) {
        const int path_idx = shuffle_ ? shard_order_[order_idx] : order_idx;
        int64_t ntok = 0;
        if (probe(paths_[path_idx], &ntok)) return -1;
        if (file_.open(paths_[path_idx])) return -1;
        current_path_ = path_idx;
        shard_samples_ = (size_t)((ntok - 1) / (int64_t)(nproc_ * B_ * T_));
        return 0;
    }
    void make_sample_order() {
        sample_order_.resize(shard_samples_);
        for (size_t i = 0; i < shard_samples_; i++) sample_order_[i] = (int)i;
        shuffle_ints(rng_, sample_order_.data(), (int)shard_samples_);
    }
    int advance() {
        if (shard_idx_ == paths_.size() - 1) return reset();
        shard_idx_ += 1;
        sample_idx_ = 0;
        if (load_shard((int)shard_idx_)) return -1;
        if (shuffle_) make_sample_order();
        return 0;
    }
    int rank_ = 0, nproc_ = 1, current_path_ = 0;
    bool shuffle_ = false;
    Mt19937 rng_;
    std::vector<int> shard_order_, sample_order_;
    MappedFile file_;
};

// ------------------------------------------------------------------------------------------ EvalLoader
// Multiple-choice eval stream (HellaSwag style): <START><BYTES><INDEX><LABEL><NCOMP><NCTX ctx..>(<N tok..>) x NCOMP,
// every field one token wide. Each example occupies 4 rows of the (B, T) batch.
class EvalLoader {
public:
    static constexpr int kCompletions = 4;
    int init(const char* path, size_t B, size_t T, int rank, int nproc) {
        B_ = B; T_ = T; rank_ = rank; nproc_ = nproc;
        if (file_.open(path)) return -1;
        if (file_.size() < kHeaderBytes) return fail("short eval file");
        const int32_t* hdr = (const int32_t*)file_.data();
        if (hdr[0] == 20240522 && hdr[1] == 1) { tb_ = 2; start_marker_ = 0xffffu; }
        else if (hdr[0] == 20240802 && hdr[1] == 7) { tb_ = 4; start_marker_ = 0xffffffffu; }
        else return fail("bad magic/version in eval file (expected 20240522 v1 or 20240802 v7)");
        num_examples_ = hdr[2];
        if (num_examples_ < nproc) return fail("fewer eval examples than processes");
        if (B_ / kCompletions == 0) return fail("eval loader needs a batch size of at least 4");
        return reset();
    }
    int reset() {
        const int per_proc = (num_examples_ + nproc_ - 1) / nproc_;
        const int fit = (int)(B_ / kCompletions);
        num_batches_ = (per_proc + fit - 1) / fit;
        start_ = per_proc * rank_;
        end_ = std::min(per_proc * (rank_ + 1), num_examples_);
        pos_ = kHeaderBytes;
        for (int i = 0; i < start_; i++) {
            uint32_t h[3];
            if (read_fields(pos_, h, 3)) return -1;
            if (h[0] != start_marker_ || h[2] != (uint32_t)i) return fail("corrupt eval example header");
            pos_ += h[1];
        }
        current_ = start_;
        return 0;
    }
    int next(int32_t* inputs, int32_t* targets, int8_t* mask, int32_t* label) {
        memset(mask, 0, B_ * T_);
        const int fit = (int)(B_ / kCompletions);
        for (int i = 0; i < fit; i++) label[i] = -1;
        for (int i = 0; i < fit && current_ < end_; i++) {
            if (next_example(i, inputs, targets, mask, label)) return -1;
        }
        return 0;
    }
    int num_examples_ = 0, num_batches_ = 0, start_ = 0, end_ = 0, current_ = 0;

private:
    uint32_t tok(size_t byte_off) const {
        return tb_ == 2 ? (uint32_t)(*(const uint16_t*)(file_.data() + byte_off)) : *(const uint32_t*)(file_.data() + byte_off);
    }
    int read_fields(size_t off, uint32_t* out, int n) const {
        if (off + (size_t)n * tb_ > file_.size()) return fail("eval file truncated");
        for (int i = 0; i < n; i++) out[i] = tok(off + (size_t)i * tb_);
        return 0;
    }
    int next_example(int slot, int32_t* inputs, int32_t* targets, int8_t* mask, int32_t* label) {
        uint32_t h[3];
        if (read_fields(pos_, h, 3)) return -1;
        if (h[0] != start_marker_ || h[2] != (uint32_t)current_) return fail("corrupt eval example header");
        const size_t ex_end = pos_ + h[1];
        if (ex_end > file_.size()) return fail("eval example runs past the file");
        size_t p = pos_ + 3 * (size_t)tb_;
        const int lab = (int)tok(p), ncomp = (int)tok(p + tb_), nctx = (int)tok(p + 2 * (size_t)tb_);
        if (lab < 0 || lab >= kCompletions || ncomp != kCompletions) return fail("unsupported eval example (label / completions)");
        if (nctx <= 0 || (size_t)nctx >= T_) return fail("eval context does not fit in T");
        label[slot] = lab;
        p += 3 * (size_t)tb_;
        const size_t row0 = (size_t)slot * kCompletions;
        for (int c = 0; c < kCompletions; c++)
            for (int i = 0; i < nctx; i++) inputs[(row0 + c) * T_ + i] = (int32_t)tok(p + (size_t)i * tb_);
        p += (size_t)nctx * tb_;
        for (int c = 0; c < kCompletions; c++) {
            const int n = (int)tok(p);
            p += tb_;
            if (n <= 0 || (size_t)(nctx + n) >= T_) return fail("eval completion does not fit in T");
            for (int i = 0; i < n; i++) {
                const int32_t t = (int32_t)tok(p + (size_t)i * tb_);
                inputs[(row0 + c) * T_ + nctx + i] = t;
                targets[(row0 + c) * T_ + nctx + i - 1] = t;
                mask[(row0 + c) * T_ + nctx + i - 1] = 1;
            }
            p += (size_t)n * tb_;
        }
        pos_ = ex_end;
        current_ += 1;
        return 0;
    }
    size_t B_ = 0, T_ = 0, pos_ = 0;
    int rank_ = 0, nproc_ = 1, tb_ = 2;
    uint32_t start_marker_ = 0xffffu;
    MappedFile file_;
};

// ------------------------------------------------------------------------------------------ Tokenizer
class Tokenizer {
public:
    int init(const char* path) {
        FILE* f = fopen(path, "rb");
        if (!f) return fail(std::string("cannot open tokenizer file ") + path);
        uint32_t hdr[kHeaderInts];
        if (fread(hdr, 4, kHeaderInts, f) != (size_t)kHeaderInts || hdr[0] != 20240328u) {
            fclose(f);
            return fail("bad tokenizer header");
        }
        const uint32_t version = hdr[1];
        const uint32_t n = hdr[2];
        eot_ = version == 1 ? 50256 : (int)hdr[3];
        if (version != 1 && version != 2) {
            fclose(f);
            return fail("unsupported tokenizer version");
        }
        table_.resize(n);
        for (uint32_t i = 0; i < n; i++) {
            uint8_t len;
            if (fread(&len, 1, 1, f) != 1) { fclose(f); return fail("truncated tokenizer file"); }
            table_[i].resize(len);
            if (len && fread(&table_[i][0], 1, len, f) != len) { fclose(f); return fail("truncated tokenizer file"); }
        }
        fclose(f);
        return 0;
    }
    std::vector<std::string> table_;
    int eot_ = 50256;
};

}  // namespace

// ================================================================================================ C API
HOST_API const char* llmk_host_last_error() { return g_error.c_str(); }

// ---- random numbers
HOST_API void* llmk_rng_create(uint32_t seed) { return new Mt19937(seed); }
HOST_API void llmk_rng_destroy(void* h) { delete (Mt19937*)h; }
HOST_API void llmk_rng_seed(void* h, uint32_t seed) { ((Mt19937*)h)->reseed(seed); }
HOST_API uint32_t llmk_rng_u32(void* h) { return ((Mt19937*)h)->next_u32(); }
HOST_API void llmk_rng_uniform(void* h, float* out, long n, float lo, float hi) {
    Mt19937& g = *(Mt19937*)h;
    for (long i = 0; i < n; i++) out[i] = g.next_f32() * (hi - lo) + lo;
}
HOST_API void llmk_rng_normal(void* h, float* out, long n, float mean, float std) { normal_fill(*(Mt19937*)h, out, (size_t)n, mean, std); }
HOST_API void llmk_rng_permutation(void* h, int* data, int n) { shuffle_ints(*(Mt19937*)h, data, n); }
HOST_API long llmk_rng_state_bytes() { return (long)Mt19937::kStateBytes; }
HOST_API void llmk_rng_save(void* h, uint8_t* out) { ((Mt19937*)h)->save(out); }
HOST_API void llmk_rng_load(void* h, const uint8_t* in) { ((Mt19937*)h)->load(in); }

// xorshift* stream used for per-step seeds and sampling (same recurrence as the reference's sampler.h:10-20)
HOST_API uint32_t llmk_xorshift_u32(uint64_t* state) {
    *state ^= *state >> 12;
    *state ^= *state << 25;
    *state ^= *state >> 27;
    return (uint32_t)((*state * 0x2545F4914F6CDD1Dull) >> 32);
}
HOST_API float llmk_xorshift_f32(uint64_t* state) { return (float)(llmk_xorshift_u32(state) >> 8) / 16777216.0f; }
// index sampled from softmax(logits) given a uniform `coin` in [0,1)
HOST_API int llmk_sample_softmax(const float* logits, int n, float coin) {
    double norm = 0.0;
    for (int i = 0; i < n; i++) norm += expf(logits[i]);
    const float target = (float)(coin * norm);
    float cdf = 0.f;
    for (int i = 0; i < n; i++) {
        cdf += expf(logits[i]);
        if (target < cdf) return i;
    }
    return n - 1;
}

// ---- data loader
HOST_API void* llmk_loader_create(const char* pattern, long B, long T, int rank, int nproc, int shuffle) {
    DataLoader* l = new DataLoader();
    if (l->init(pattern, (size_t)B, (size_t)T, rank, nproc, shuffle)) {
        delete l;
        return nullptr;
    }
    return l;
}
HOST_API void llmk_loader_destroy(void* h) { delete (DataLoader*)h; }
HOST_API int llmk_loader_next(void* h, int32_t* inputs, int32_t* targets) { return ((DataLoader*)h)->next(inputs, targets); }
HOST_API int llmk_loader_reset(void* h) { return ((DataLoader*)h)->reset(); }
HOST_API int llmk_loader_resume(void* h, long shard_idx, long sample_idx) { return ((DataLoader*)h)->resume((size_t)shard_idx, (size_t)sample_idx); }
HOST_API long llmk_loader_num_tokens(void* h) { return (long)((DataLoader*)h)->num_tokens_; }
HOST_API long llmk_loader_shard_idx(void* h) { return (long)((DataLoader*)h)->shard_idx_; }
HOST_API long llmk_loader_sample_idx(void* h) { return (long)((DataLoader*)h)->sample_idx_; }
HOST_API long llmk_loader_shard_samples(void* h) { return (long)((DataLoader*)h)->shard_samples_; }
HOST_API int llmk_loader_num_shards(void* h) { return (int)((DataLoader*)h)->paths_.size(); }
HOST_API int llmk_loader_token_bytes(void* h) { return ((DataLoader*)h)->token_bytes_; }
HOST_API long llmk_loader_shuffle_state_bytes(void* h) { return (long)((DataLoader*)h)->shuffle_state_bytes(); }
HOST_API void llmk_loader_save_shuffle_state(void* h, uint8_t* out) { ((DataLoader*)h)->save_shuffle_state(out); }
HOST_API int llmk_loader_load_shuffle_state(void* h, const uint8_t* in, long n) { return ((DataLoader*)h)->load_shuffle_state(in, (size_t)n); }

// ---- eval loader
HOST_API void* llmk_evalloader_create(const char* path, long B, long T, int rank, int nproc) {
    EvalLoader* l = new EvalLoader();
    if (l->init(path, (size_t)B, (size_t)T, rank, nproc)) {
        delete l;
        return nullptr;
    }
    return l;
}
HOST_API void llmk_evalloader_destroy(void* h) { delete (EvalLoader*)h; }
HOST_API int llmk_evalloader_reset(void* h) { return ((EvalLoader*)h)->reset(); }
HOST_API int llmk_evalloader_next(void* h, int32_t* inputs, int32_t* targets, int8_t* mask, int32_t* label) {
    return ((EvalLoader*)h)->next(inputs, targets, mask, label);
}
HOST_API int llmk_evalloader_num_examples(void* h) { return ((EvalLoader*)h)->num_examples_; }
HOST_API int llmk_evalloader_num_batches(void* h) { return ((EvalLoader*)h)->num_batches_; }
// number of examples of the batch whose lowest mean masked loss is the labelled completion
HOST_API int llmk_evalloader_stat_losses(const float* losses, const int8_t* mask, const int32_t* label, long B, long T) {
    int correct = 0;
    for (long ex = 0; ex < B / 4; ex++) {
        float best = 0.f;
        int best_idx = -1;
        bool active = false;
        for (int c = 0; c < 4; c++) {
            const long row = ex * 4 + c;
            float sum = 0.f;
            int cnt = 0;
            for (long t = 0; t < T; t++) {
                if (mask[row * T + t] == 1) {
                    active = true;
                    sum += losses[row * T + t];
                    cnt++;
                }
            }
            const float avg = cnt > 0 ? sum / cnt : 0.f;
            if (c == 0 || avg < best) {
                best = avg;
                best_idx = c;
            }
        }
        if (active && best_idx == label[ex]) correct++;
    }
    return correct;
}

// ---- tokenizer
HOST_API void* llmk_tokenizer_create(const char* path) {
    Tokenizer* t = new Tokenizer();
    if (t->init(path)) {
        delete t;
        return nullptr;
    }
    return t;
}
HOST_API void llmk_tokenizer_destroy(void* h) { delete (Tokenizer*)h; }
HOST_API int llmk_tokenizer_vocab_size(void* h) { return (int)((Tokenizer*)h)->table_.size(); }
HOST_API int llmk_tokenizer_eot(void* h) { return ((Tokenizer*)h)->eot_; }
// copies the bytes of token `id` into out (up to cap) and returns the token's length, or -1
HOST_API int llmk_tokenizer_decode(void* h, int id, uint8_t* out, int cap) {
    Tokenizer* t = (Tokenizer*)h;
    if (id < 0 || id >= (int)t->table_.size()) return -1;
    const std::string& s = t->table_[id];
    const int n = (int)std::min<size_t>(s.size(), (size_t)cap);
    memcpy(out, s.data(), n);
    return (int)s.size();
}

// ---- learning-rate schedules (cosine, linear, constant, wsd) with linear warm-up (step + 1) / warmup; float32
// arithmetic, the same curves as llmc/schedulers.h:19-98 of the reference. kind: 0 cosine, 1 linear, 2 constant, 3 wsd.
// Returns NaN for a step beyond the schedule or an unknown kind.
HOST_API float llmk_lr_get(int kind, float lr, int warmup, int total, float final_frac, int step) {
    const float min_lr = lr * final_frac;
    if (kind == 2) return lr;
    if (kind < 0 || kind > 3) return NAN;
    if (step < warmup) return lr * (float)(step + 1) / (float)warmup;
    if (kind == 3) {
        const int decay_point = (int)(0.8f * (float)total);
        if (step < decay_point) return lr;
        const float ratio = (float)(step - decay_point) / (float)(total - decay_point);
        return min_lr + (1.0f - sqrtf(ratio)) * (lr - min_lr);
    }
    const float ratio = (float)(step - warmup) / (float)(total - warmup);
    if (!(ratio >= 0.0f && ratio <= 1.0f)) return NAN;
    if (kind == 0) {
        const float coeff = 0.5f * (1.0f + cosf((float)M_PI * ratio));
        return min_lr + coeff * (lr - min_lr);
    }
    return lr - ratio * (lr - min_lr);
}

// ---- outlier detector: z-score of a value against the previous 128 (double precision running sums); NaN until the
// window is full (llmc/outlier_detector.h:16-70)
struct OutlierDetector {
    static constexpr int WINDOW = 128;
    double buffer[WINDOW];
    int count = 0, index = 0;
    double sum = 0.0, sum_sq = 0.0;
    double update(double v) {
        if (count < WINDOW) {
            buffer[count++] = v;
            sum += v;
            sum_sq += v * v;
            return NAN;
        }
        const double old = buffer[index];
        sum += v - old;
        sum_sq += v * v - old * old;
        buffer[index] = v;
        index = (index + 1) % WINDOW;
        const double mean = sum / WINDOW;
        const double var = sum_sq / WINDOW - mean * mean;
        const double sd = var > 0 ? sqrt(var) : 0.0;
        return sd == 0.0 ? 0.0 : (v - mean) / sd;
    }
};
HOST_API void* llmk_outlier_create() { return new OutlierDetector(); }
HOST_API void llmk_outlier_destroy(void* h) { delete (OutlierDetector*)h; }
HOST_API double llmk_outlier_update(void* h, double v) { return ((OutlierDetector*)h)->update(v); }

// ---- logger: rank 0's main.log, opened per line in append mode (a crash loses nothing), wiped at creation unless
// resuming; line formats as in llmc/logger.h:19-56 because log validators parse them
struct HostLogger {
    std::string path;
    bool active = false;
    void line(const char* text) {
        if (!active) return;
        FILE* f = fopen(path.c_str(), "a");
        if (f == nullptr) return;
        fputs(text, f);
        fclose(f);
    }
};
HOST_API void* llmk_logger_create(const char* dir, int rank, int resume) {
    HostLogger* l = new HostLogger();
    if (dir != nullptr && dir[0] != 0 && rank == 0) {
        l->active = true;
        l->path = std::string(dir) + "/main.log";
        if (!resume) {
            FILE* f = fopen(l->path.c_str(), "w");
            if (f != nullptr) fclose(f);
        }
    }
    return l;
}
HOST_API void llmk_logger_destroy(void* h) { delete (HostLogger*)h; }
HOST_API void llmk_logger_eval(void* h, int step, float val) {
    char buf[128];
    snprintf(buf, sizeof buf, "s:%d eval:%.4f\n", step, val);
    ((HostLogger*)h)->line(buf);
}
HOST_API void llmk_logger_val(void* h, int step, float val_loss) {
    char buf[128];
    snprintf(buf, sizeof buf, "s:%d tel:%.4f\n", step, val_loss);
    ((HostLogger*)h)->line(buf);
}
HOST_API void llmk_logger_train(void* h, int step, float train_loss, float lr, float grad_norm) {
    char buf[160];
    snprintf(buf, sizeof buf, "s:%d trl:%.4f lr:%.6f norm:%.2f\n", step, train_loss, lr, grad_norm);
    ((HostLogger*)h)->line(buf);
}
