// Native latency harness for the small shapes the reference publishes numbers for, driven through
// the C ABI only (no Python in the timed region).
//
// Protocol = the reference's `eager_stream_batch_cuda_event`
// (crates/loom-infer-validation/src/benchmarks/matched.rs:141-173): plan, allocation and upload
// outside; 200 warm-up calls; per sample one CUDA-event pair around 100 provider calls enqueued in
// ONE command scope on one stream, divided by 100; median of the samples.  Host submission gaps
// are included, as in the reference.  A second figure times the same 100 calls captured as one
// fixed-address Graph (device time per call without host launch cost), and a third one Graph of
// a single call plus its completion event (crates/loom-infer-cuda/src/graph/mod.rs:301-323).
//
//     loom_native_bench [--samples 50] [--calls 100] [--device 0] [--only <part of a case name>]
//
// Prints one JSON object per case.
#include <cuda_runtime.h>

#include <algorithm>
#include <chrono>
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>

#include "loom_b200.h"

namespace {

[[noreturn]] void die(const char *what, int code) {
    lb_error_info info;
    lb_last_error(&info);
    std::fprintf(stderr, "%s failed: %d (%s)\n", what, code, lb_status_name(code));
    std::exit(1);
}
#define LB(call)                                                                                   \
    do {                                                                                           \
        const lb_status status_ = (call);                                                          \
        if (status_ != 0) die(#call, status_);                                                     \
    } while (0)
#define CU(call)                                                                                   \
    do {                                                                                           \
        const cudaError_t error_ = (call);                                                         \
        if (error_ != cudaSuccess) {                                                               \
            std::fprintf(stderr, "%s: %s\n", #call, cudaGetErrorString(error_));                   \
            std::exit(1);                                                                          \
        }                                                                                          \
    } while (0)

// xorshift64* -> roughly N(0,1) BF16 bits (sum of four uniforms), seeded per buffer
struct Rng {
    uint64_t state;
    explicit Rng(uint64_t seed) : state(seed * 0x9E3779B97F4A7C15ull + 1) {}
    double uniform() {
        state ^= state >> 12;
        state ^= state << 25;
        state ^= state >> 27;
        return (double)((state * 0x2545F4914F6CDD1Dull) >> 11) / 9007199254740992.0;
    }
    uint16_t normal_bf16() {
        const float x = (float)((uniform() + uniform() + uniform() + uniform() - 2.0) * 1.7320508);
        uint32_t bits;
        std::memcpy(&bits, &x, 4);
        bits += 0x7fffu + ((bits >> 16) & 1u);
        return (uint16_t)(bits >> 16);
    }
};

template <typename T> T *upload(const std::vector<T> &host) {
    T *device = nullptr;
    CU(cudaMalloc(&device, std::max<size_t>(host.size(), 1) * sizeof(T)));
    if (!host.empty())
        CU(cudaMemcpy(device, host.data(), host.size() * sizeof(T), cudaMemcpyHostToDevice));
    return device;
}
uint16_t *upload_normal(size_t numel, uint64_t seed) {
    Rng rng(seed);
    std::vector<uint16_t> host(numel);
    for (auto &x : host) x = rng.normal_bf16();
    return upload(host);
}
template <typename T> T *device_zeros(size_t numel) {
    T *device = nullptr;
    CU(cudaMalloc(&device, std::max<size_t>(numel, 1) * sizeof(T)));
    CU(cudaMemset(device, 0, std::max<size_t>(numel, 1) * sizeof(T)));
    return device;
}

double median(std::vector<double> values) {
    std::sort(values.begin(), values.end());
    const size_t n = values.size();
    return n % 2 ? values[n / 2] : 0.5 * (values[n / 2 - 1] + values[n / 2]);
}

// One benchmarked operation: binds its buffers into a bindings set and enqueues one call.
struct Case {
    std::string name;
    size_t slots = 0, commands = 1;
    virtual void bind(lb_bindings *bindings) = 0;
    virtual lb_status enqueue(lb_scope *scope) = 0;
    virtual ~Case() = default;
};

struct Options {
    int samples = 50, calls = 100, device = 0;
    std::string only; // run only the cases whose name contains this
};

lb_status record_calls(lb_scope *scope, void *user) {
    auto *pair = static_cast<std::pair<Case *, int> *>(user);
    for (int i = 0; i < pair->second; ++i) {
        const lb_status rc = pair->first->enqueue(scope);
        if (rc) return rc;
    }
    return 0;
}

void measure(Case &c, const Options &opt) {
    cudaStream_t stream;
    CU(cudaStreamCreate(&stream));
    lb_queue *queue = nullptr;
    LB(lb_queue_create(stream, (size_t)opt.calls * c.commands + 1, &queue));
    lb_bindings *bindings = nullptr;
    LB(lb_queue_bindings(queue, c.slots, &bindings));
    c.bind(bindings);
    auto run_scope = [&](int calls) {
        lb_scope *scope = nullptr;
        LB(lb_queue_begin(queue, bindings, &scope));
        for (int i = 0; i < calls; ++i) LB(c.enqueue(scope));
        lb_completion *completion = nullptr;
        LB(lb_scope_finish(scope, &completion));
        return completion;
    };
    for (int i = 0; i < 2; ++i) LB(lb_completion_wait(run_scope(opt.calls), &bindings));
    cudaEvent_t start, end;
    CU(cudaEventCreate(&start));
    CU(cudaEventCreate(&end));
    std::vector<double> eager, host;
    for (int s = 0; s < opt.samples; ++s) {
        CU(cudaEventRecord(start, stream));
        const auto host_start = std::chrono::steady_clock::now();
        lb_scope *scope = nullptr;
        LB(lb_queue_begin(queue, bindings, &scope));
        for (int i = 0; i < opt.calls; ++i) LB(c.enqueue(scope));
        host.push_back(std::chrono::duration<double, std::micro>(
                           std::chrono::steady_clock::now() - host_start).count() / opt.calls);
        CU(cudaEventRecord(end, stream));
        lb_completion *completion = nullptr;
        LB(lb_scope_finish(scope, &completion));
        LB(lb_completion_wait(completion, &bindings));
        float ms = 0.0f;
        CU(cudaEventElapsedTime(&ms, start, end));
        eager.push_back(ms * 1e3 / opt.calls);
    }
    lb_bindings_destroy(bindings);
    lb_queue_destroy(queue);

    // fixed-address Graphs: `calls` calls in one Graph, and one call per Graph
    double graph_batch = 0.0, graph_single = 0.0;
    for (int variant = 0; variant < 2; ++variant) {
        const int calls = variant == 0 ? opt.calls : 1;
        lb_graph_queue *gq = nullptr;
        LB(lb_graph_queue_create(opt.device, (size_t)calls * c.commands + 1, &gq));
        lb_bindings *gb = nullptr;
        LB(lb_graph_queue_bindings(gq, c.slots, &gb));
        c.bind(gb);
        std::pair<Case *, int> user(&c, calls);
        lb_captured_graph *graph = nullptr;
        LB(lb_graph_capture(gq, gb, record_calls, &user, &graph));
        lb_graph_exec *exec = nullptr;
        LB(lb_captured_graph_instantiate(graph, &exec));
        std::vector<double> times;
        for (int s = 0; s < opt.samples + 5; ++s) {
            float ms = 0.0f;
            LB(lb_graph_exec_measure_launch_ms(exec, &ms));
            if (s >= 5) times.push_back(ms * 1e3 / calls);
        }
        (variant == 0 ? graph_batch : graph_single) = median(times);
        lb_bindings *back = nullptr; // capture moved the queue and the bindings into the graph
        LB(lb_graph_exec_into_bindings(exec, &back));
        lb_bindings_destroy(back);
    }
    std::vector<double> sorted = eager;
    std::sort(sorted.begin(), sorted.end());
    std::printf("{\"provider\": \"loom_b200\", \"harness\": \"native C ABI\", \"case\": \"%s\", "
                "\"measurement\": \"eager_stream_batch_cuda_event\", \"launches_per_sample\": %d, "
                "\"samples\": %d, \"commands_per_call\": %zu, \"us_per_call\": %.3f, "
                "\"p10_us\": %.3f, \"p90_us\": %.3f, \"host_submit_us_per_call\": %.3f, "
                "\"graph_batch_us_per_call\": %.3f, "
                "\"graph_single_us\": %.3f}\n",
                c.name.c_str(), opt.calls, opt.samples, c.commands, median(eager),
                sorted[sorted.size() / 10], sorted[sorted.size() * 9 / 10], median(host),
                graph_batch,
                graph_single);
    std::fflush(stdout);
    CU(cudaEventDestroy(start));
    CU(cudaEventDestroy(end));
    CU(cudaStreamDestroy(stream));
}

struct DecodeCase : Case {
    lb_paged_spec spec{};
    lb_paged_decode_plan *plan = nullptr;
    uint16_t *query, *key_pages, *value_pages, *output;
    int32_t *indptr, *indices, *last;
    float *lse, *workspace = nullptr;
    size_t indices_len, workspace_numel = 0;
    lb_paged_decode_args args{};

    DecodeCase(const char *label, lb_decode_provider *provider, size_t batch, size_t pages,
               size_t qh, size_t kvh, std::vector<int32_t> page_indptr,
               std::vector<int32_t> page_indices, std::vector<int32_t> last_page_len,
               uint32_t partitions, const lb_paged_decode_options *pinned = nullptr) {
        name = label;
        LB(lb_paged_spec_new(batch, pages, qh, kvh, 128, 16, &spec));
        lb_paged_decode_options options{};
        options.partitions = partitions;
        if (pinned) options = *pinned;
        LB(lb_paged_decode_plan_create(provider, &spec, &options, &plan));
        lb_paged_decode_plan_info info{};
        LB(lb_paged_decode_plan_info_get(plan, nullptr, &info));
        commands = info.commands;
        workspace_numel = info.workspace_numel;
        indices_len = page_indices.size();
        query = upload_normal(lb_paged_spec_query_numel(&spec), 1);
        key_pages = upload_normal(lb_paged_spec_kv_pages_numel(&spec), 2);
        value_pages = upload_normal(lb_paged_spec_kv_pages_numel(&spec), 3);
        output = device_zeros<uint16_t>(lb_paged_spec_query_numel(&spec));
        lse = device_zeros<float>(lb_paged_spec_lse_numel(&spec));
        if (workspace_numel) workspace = device_zeros<float>(workspace_numel);
        indptr = upload(page_indptr);
        indices = upload(page_indices);
        last = upload(last_page_len);
        slots = 9;
    }
    void bind(lb_bindings *b) override {
        lb_handle out{}, l{}, ws{};
        LB(lb_bind_read(b, LB_BF16, query, lb_paged_spec_query_numel(&spec), &args.query));
        LB(lb_bind_read(b, LB_BF16, key_pages, lb_paged_spec_kv_pages_numel(&spec),
                        &args.key_pages));
        LB(lb_bind_read(b, LB_BF16, value_pages, lb_paged_spec_kv_pages_numel(&spec),
                        &args.value_pages));
        LB(lb_bind_read(b, LB_I32, indptr, spec.batch_size + 1, &args.page_indptr));
        LB(lb_bind_read(b, LB_I32, indices, indices_len, &args.page_indices));
        LB(lb_bind_read(b, LB_I32, last, spec.batch_size, &args.last_page_len));
        LB(lb_bind_read_write(b, LB_BF16, output, lb_paged_spec_query_numel(&spec), &out));
        LB(lb_bind_read_write(b, LB_F32, lse, lb_paged_spec_lse_numel(&spec), &l));
        args.output = lb_handle_write(out);
        args.lse = lb_handle_write(l);
        args.workspace = lb_handle{};
        if (workspace_numel) {
            LB(lb_bind_read_write(b, LB_F32, workspace, workspace_numel, &ws));
            args.workspace = ws;
        }
    }
    lb_status enqueue(lb_scope *scope) override {
        return lb_paged_decode_enqueue(plan, scope, &args);
    }
};

struct AppendCase : Case {
    lb_paged_spec spec{};
    lb_rope_append_plan *plan = nullptr;
    size_t tokens, indices_len;
    uint16_t *query, *key, *value, *query_output, *key_pages, *value_pages;
    int32_t *batch_indices, *positions, *indptr, *indices, *last;
    lb_rope_append_args args{};
    int32_t *workspace = nullptr; // extended plans: the validation's verdicts and slots
    size_t workspace_numel = 0;

    // request r appends new_tokens[r] tokens after prior[r] existing ones; pages in order.
    // extended: no 64-token cap on the call (validate and scatter as two commands, or as one)
    AppendCase(const char *label, lb_rope_provider *provider, size_t pool_pages, size_t qh,
               size_t kvh, const std::vector<int> &new_tokens, const std::vector<int> &prior,
               bool extended = false, bool one_command = false) {
        name = label;
        const size_t batch = new_tokens.size();
        std::vector<int32_t> page_indptr{0}, page_indices, last_page_len, owner, position;
        int next_page = 0;
        for (size_t r = 0; r < batch; ++r) {
            const int len = prior[r] + new_tokens[r];
            for (int p = 0; p < (len + 15) / 16; ++p) page_indices.push_back(next_page++);
            page_indptr.push_back((int32_t)page_indices.size());
            last_page_len.push_back((len - 1) % 16 + 1);
            for (int t = 0; t < new_tokens[r]; ++t) {
                owner.push_back((int32_t)r);
                position.push_back(prior[r] + t);
            }
        }
        tokens = owner.size();
        indices_len = page_indices.size();
        lb_append_tokens_spec token_spec{};
        if (extended)
            LB(lb_append_tokens_spec_new_extended(tokens, batch, pool_pages, qh, kvh, 128, 16,
                                                  &token_spec));
        else
            LB(lb_append_tokens_spec_new(tokens, batch, pool_pages, qh, kvh, 128, 16, &token_spec));
        LB(lb_paged_spec_new(batch, pool_pages, qh, kvh, 128, 16, &spec));
        lb_rope_append_options options{};
        options.one_command = one_command ? 1 : 0;
        LB(lb_rope_append_tokens_plan_create_with(provider, &token_spec, &options, &plan));
        lb_rope_append_plan_info info{};
        LB(lb_rope_append_plan_info_get(plan, &info));
        commands = (int)info.commands;
        workspace_numel = info.workspace_numel;
        if (workspace_numel) workspace = device_zeros<int32_t>(workspace_numel);
        query = upload_normal(tokens * qh * 128, 4);
        key = upload_normal(tokens * kvh * 128, 5);
        value = upload_normal(tokens * kvh * 128, 6);
        query_output = device_zeros<uint16_t>(tokens * qh * 128);
        key_pages = device_zeros<uint16_t>(lb_paged_spec_kv_pages_numel(&spec));
        value_pages = device_zeros<uint16_t>(lb_paged_spec_kv_pages_numel(&spec));
        batch_indices = upload(owner);
        positions = upload(position);
        indptr = upload(page_indptr);
        indices = upload(page_indices);
        last = upload(last_page_len);
        slots = 12;
    }
    void bind(lb_bindings *b) override {
        const size_t qh = spec.num_query_heads, kvh = spec.num_kv_heads;
        lb_handle q_out{}, kp{}, vp{};
        if (workspace_numel)
            LB(lb_bind_read_write(b, LB_I32, workspace, workspace_numel, &args.workspace));
        LB(lb_bind_read(b, LB_BF16, query, tokens * qh * 128, &args.query));
        LB(lb_bind_read(b, LB_BF16, key, tokens * kvh * 128, &args.key));
        LB(lb_bind_read(b, LB_BF16, value, tokens * kvh * 128, &args.value));
        LB(lb_bind_read(b, LB_I32, batch_indices, tokens, &args.batch_indices));
        LB(lb_bind_read(b, LB_I32, positions, tokens, &args.positions));
        LB(lb_bind_read(b, LB_I32, indptr, spec.batch_size + 1, &args.page_indptr));
        LB(lb_bind_read(b, LB_I32, indices, indices_len, &args.page_indices));
        LB(lb_bind_read(b, LB_I32, last, spec.batch_size, &args.last_page_len));
        LB(lb_bind_read_write(b, LB_BF16, query_output, tokens * qh * 128, &q_out));
        LB(lb_bind_read_write(b, LB_BF16, key_pages, lb_paged_spec_kv_pages_numel(&spec), &kp));
        LB(lb_bind_read_write(b, LB_BF16, value_pages, lb_paged_spec_kv_pages_numel(&spec), &vp));
        args.query_output = lb_handle_write(q_out);
        args.key_pages = lb_handle_write(kp);
        args.value_pages = lb_handle_write(vp);
    }
    lb_status enqueue(lb_scope *scope) override {
        return lb_rope_append_enqueue(plan, scope, &args);
    }
};

// Paged causal prefill: requests with qo_lens[r] query tokens over kv_lens[r] KV tokens, pages in
// a fixed scattered order.
struct PrefillCase : Case {
    lb_prefill_spec spec{};
    lb_paged_prefill_plan *plan = nullptr;
    uint16_t *query, *key_pages, *value_pages, *output;
    int32_t *qo_indptr, *indptr, *indices, *last;
    float *lse;
    size_t indices_len;
    lb_paged_prefill_args args{};

    PrefillCase(const char *label, lb_prefill_provider *provider, size_t qh, size_t kvh,
                const std::vector<int> &qo_lens, const std::vector<int> &kv_lens) {
        name = label;
        const size_t batch = qo_lens.size();
        std::vector<int32_t> qo{0}, page_indptr{0}, page_indices, last_page_len;
        size_t total_pages = 0;
        for (size_t r = 0; r < batch; ++r) total_pages += (size_t)(kv_lens[r] + 15) / 16;
        const size_t pool = total_pages + 8;
        size_t next = 0, stride = 37; // a stride coprime to the pool visits every page once
        auto gcd = [](size_t x, size_t y) { while (y) { const size_t t = x % y; x = y; y = t; } return x; };
        while (gcd(stride, pool) != 1) ++stride;
        for (size_t r = 0; r < batch; ++r) {
            qo.push_back(qo.back() + qo_lens[r]);
            for (int p = 0; p < (kv_lens[r] + 15) / 16; ++p)
                page_indices.push_back((int32_t)((next++ * stride + 11) % pool));
            page_indptr.push_back((int32_t)page_indices.size());
            last_page_len.push_back((kv_lens[r] - 1) % 16 + 1);
        }
        indices_len = page_indices.size();
        LB(lb_prefill_spec_new(batch, (size_t)qo.back(), pool, qh, kvh, 128, 16, &spec));
        LB(lb_paged_prefill_plan_create(provider, &spec, nullptr, &plan));
        commands = 1;
        query = upload_normal(lb_prefill_spec_query_numel(&spec), 7);
        key_pages = upload_normal(lb_prefill_spec_kv_pages_numel(&spec), 8);
        value_pages = upload_normal(lb_prefill_spec_kv_pages_numel(&spec), 9);
        output = device_zeros<uint16_t>(lb_prefill_spec_query_numel(&spec));
        lse = device_zeros<float>(lb_prefill_spec_lse_numel(&spec));
        qo_indptr = upload(qo);
        indptr = upload(page_indptr);
        indices = upload(page_indices);
        last = upload(last_page_len);
        slots = 9;
    }
    void bind(lb_bindings *b) override {
        lb_handle out{}, l{};
        const size_t pool = lb_prefill_spec_kv_pages_numel(&spec);
        LB(lb_bind_read(b, LB_BF16, query, lb_prefill_spec_query_numel(&spec), &args.query));
        LB(lb_bind_read(b, LB_BF16, key_pages, pool, &args.key_pages));
        LB(lb_bind_read(b, LB_BF16, value_pages, pool, &args.value_pages));
        LB(lb_bind_read(b, LB_I32, qo_indptr, spec.batch_size + 1, &args.qo_indptr));
        LB(lb_bind_read(b, LB_I32, indptr, spec.batch_size + 1, &args.page_indptr));
        LB(lb_bind_read(b, LB_I32, indices, indices_len, &args.page_indices));
        LB(lb_bind_read(b, LB_I32, last, spec.batch_size, &args.last_page_len));
        LB(lb_bind_read_write(b, LB_BF16, output, lb_prefill_spec_query_numel(&spec), &out));
        LB(lb_bind_read_write(b, LB_F32, lse, lb_prefill_spec_lse_numel(&spec), &l));
        args.output = lb_handle_write(out);
        args.lse = lb_handle_write(l);
    }
    lb_status enqueue(lb_scope *scope) override {
        return lb_paged_prefill_enqueue(plan, scope, &args);
    }
};

} // namespace

int main(int argc, char **argv) {
    Options opt;
    for (int i = 1; i + 1 < argc; i += 2) {
        if (!std::strcmp(argv[i], "--samples")) opt.samples = std::atoi(argv[i + 1]);
        else if (!std::strcmp(argv[i], "--calls")) opt.calls = std::atoi(argv[i + 1]);
        else if (!std::strcmp(argv[i], "--device")) opt.device = std::atoi(argv[i + 1]);
        else if (!std::strcmp(argv[i], "--only")) opt.only = argv[i + 1];
    }
    CU(cudaSetDevice(opt.device));
    lb_decode_provider *decode = nullptr;
    lb_rope_provider *rope = nullptr;
    lb_prefill_provider *prefill = nullptr;
    LB(lb_decode_provider_load(opt.device, &decode));
    LB(lb_rope_provider_load(opt.device, &rope));
    LB(lb_prefill_provider_load(opt.device, &prefill));

    // the three paged-decode shapes and the two append shapes with published reference numbers
    DecodeCase mha("gate mha_b1_l1", decode, 1, 2, 8, 8, {0, 1}, {1}, {1}, 1);
    DecodeCase mqa("gate mqa_b3_mixed", decode, 3, 7, 8, 1, {0, 1, 3, 6}, {4, 6, 1, 5, 0, 3},
                   {16, 7, 16}, 1);
    DecodeCase gqa("gate gqa4_b4_reuse", decode, 4, 8, 16, 4, {0, 1, 3, 5, 8},
                   {7, 2, 6, 5, 1, 7, 0, 4}, {3, 16, 1, 9}, 1);
    AppendCase one("gate append b4 16/4 one token per request", rope, 16, 16, 4, {1, 1, 1, 1},
                   {0, 15, 16, 40});
    AppendCase six("gate append b3 16/4 six explicit tokens", rope, 16, 16, 4, {1, 2, 3},
                   {3, 16, 30});
    // C2 of the configuration list: 32 requests, 1-64 new tokens each after 0-2048 cached ones,
    // 32/8 heads, one extended call (fixed pseudo-random lengths: 1081 tokens in all)
    std::vector<int> c2_new(32), c2_prior(32);
    for (int r = 0, total = 0; r < 32; ++r) {
        c2_new[r] = r == 31 ? 1081 - total : (r + 17) % 64 + 1; // 18 .. 48, then 58
        total += c2_new[r];
        c2_prior[r] = (r * 613 + 101) % 2049;
    }
    AppendCase c2("C2 RoPE+append b32 32/8 tokens1081 pool8192 extended", rope, 8192, 32, 8, c2_new,
                  c2_prior, true);
    AppendCase c2_one("C2 RoPE+append b32 32/8 tokens1081 pool8192 extended, as one command", rope,
                      8192, 32, 8, c2_new, c2_prior, true, true);
    // C1 of the configuration list: MHA batch 1, 32/32 heads, context 1024, plan-chosen split
    std::vector<int32_t> c1_pages(64);
    for (int i = 0; i < 64; ++i) c1_pages[i] = (i * 37 + 11) % 256;
    DecodeCase c1("C1 paged decode MHA b1 32/32 ctx1024 pool256 (plan-chosen)", decode, 1, 256, 32,
                  32, {0, 64}, c1_pages, {16}, 0);
    // the five paged-prefill shapes with published reference numbers
    PrefillCase p_mha("gate prefill mha_b1_q4_kv4 8/8", prefill, 8, 8, {4}, {4});
    PrefillCase p_mqa("gate prefill mqa_b3_q2_3_1_kv4_22_35 8/1", prefill, 8, 1, {2, 3, 1},
                      {4, 22, 35});
    PrefillCase p_gqa("gate prefill gqa4_b2_q4_2_kv23_18 16/4", prefill, 16, 4, {4, 2}, {23, 18});
    PrefillCase p_mqa_long("gate prefill mqa_b3_q1_4_16_kv128_256_512 8/1", prefill, 8, 1,
                           {1, 4, 16}, {128, 256, 512});
    PrefillCase p_gqa_long("gate prefill gqa4_b2_q32_64_kv256_1024 16/4", prefill, 16, 4, {32, 64},
                           {256, 1024});
    // C1 with the plan's parameters pinned (heads per CTA, chunks, cluster / in-kernel merge /
    // two-command split): the measurements behind the plan-time rule for a single short request
    std::vector<DecodeCase *> c1_variants;
    if (!opt.only.empty() && opt.only.find("C1") == 0) {
        // {heads per CTA, chunks, cluster, merge_in_kernel}
        const uint32_t grid[][4] = {{4, 8, 1, 0}, {4, 8, 0, 1}, {4, 16, 0, 1}, {2, 8, 0, 1},
                                    {4, 9, 0, 0}, {4, 18, 0, 0}, {1, 4, 1, 0}, {2, 8, 1, 0}};
        for (const auto &g : grid) {
            lb_paged_decode_options o{};
            o.heads_per_cta = g[0];
            o.partitions = g[1];
            o.cluster = g[2];
            o.merge_in_kernel = g[3];
            char label[160];
            std::snprintf(label, sizeof(label),
                          "C1 variant hc%u x %u chunks, %s", g[0], g[1],
                          g[2]        ? "cluster (1 command)"
                          : g[3] == 1 ? "workspace, merged by the last CTA (1 command)"
                                      : "workspace, merge command (2 commands)");
            c1_variants.push_back(new DecodeCase(label, decode, 1, 256, 32, 32, {0, 64}, c1_pages,
                                                 {16}, 0, &o));
        }
    }
    std::vector<Case *> cases = {&mha, &mqa, &gqa, &one, &six, &c2, &c2_one, &c1, &p_mha, &p_mqa, &p_gqa,
                                 &p_mqa_long, &p_gqa_long};
    for (DecodeCase *c : c1_variants) cases.push_back(c);
    for (Case *c : cases)
        if (opt.only.empty() || c->name.find(opt.only) != std::string::npos) measure(*c, opt);
    return 0;
}
