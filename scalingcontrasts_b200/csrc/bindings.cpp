// Python bindings of the native layer. Pointers cross as integers (device addresses, possibly inside symmetric
// memory that torch does not own), streams as the integer handle torch reports; the Python wrappers validate shapes,
// dtypes and contiguity before calling in.
#include <torch/extension.h>

#include <atomic>
#include <memory>

#include "api.h"
#include "domain.h"
#include "rail.h"

namespace py = pybind11;

namespace sc {

namespace {
std::atomic<uint64_t> launches{0};
}
uint64_t launch_count() { return launches.load(); }
void note_launch(uint64_t count) { launches.fetch_add(count); }

} // namespace sc

namespace {

template <typename T>
T* pointer(uint64_t address) {
    return reinterpret_cast<T*>(static_cast<uintptr_t>(address));
}
cudaStream_t stream_of(uint64_t handle) { return reinterpret_cast<cudaStream_t>(static_cast<uintptr_t>(handle)); }

sc::ladder_host ladder_of(std::vector<uint32_t> const& ends) {
    if (ends.empty() || ends.size() > sc::max_prefixes) throw std::runtime_error("a ladder holds 1..8 prefixes");
    sc::ladder_host ladder{};
    ladder.count = static_cast<uint32_t>(ends.size());
    for (size_t i = 0; i < ends.size(); ++i) ladder.ends[i] = ends[i];
    return ladder;
}

// Byte offsets of the control words inside a replica's control block.
constexpr uint64_t control_flag = 0, control_round = 16, control_finished = 32, control_status = 64;

struct control_handle {
    sc::control_view view{};
    std::vector<void*> replicas; // every member's replica base, for the peer path
    uint64_t multicast_base = 0;
    uint64_t own_base = 0;
};

std::shared_ptr<control_handle> make_control(sc::native_domain const& domain, uint64_t control_offset, uint64_t budget_ns,
                                             bool use_multicast) {
    auto handle = std::make_shared<control_handle>();
    uint64_t const own = domain.replica(domain.member()) + control_offset;
    handle->view.own_flag = pointer<uint32_t>(own + control_flag);
    handle->view.own_round = pointer<uint32_t>(own + control_round);
    handle->view.own_finished = pointer<uint32_t>(own + control_finished);
    handle->view.status = pointer<uint32_t>(own + control_status);
    handle->view.multicast_flag =
        use_multicast && domain.has_multicast() ? pointer<uint32_t>(domain.multicast() + control_offset + control_flag) : nullptr;
    handle->view.members = static_cast<uint32_t>(domain.members());
    handle->view.member = static_cast<uint32_t>(domain.member());
    handle->view.budget_ns = budget_ns;
    for (int m = 0; m < domain.members(); ++m) {
        handle->view.peer_flags[m] = pointer<uint32_t>(domain.replica(m) + control_offset + control_flag);
        handle->replicas.push_back(pointer<void>(domain.replica(m)));
    }
    handle->multicast_base = use_multicast && domain.has_multicast() ? domain.multicast() : 0;
    handle->own_base = domain.replica(domain.member());
    return handle;
}

// Everything about a streamed-loss object that does not change from block to block, so that scoring a block is one
// call from Python: the transpose, the tile kernel(s) and the fold of the partial sums are enqueued here back to back.
void runtime_check(cudaError_t result, char const* what) {
    if (result != cudaSuccess) throw std::runtime_error(std::string(what) + " failed: " + cudaGetErrorString(result));
}

struct loss_plan {
    uint32_t rows_q = 0, rows_c = 0, hidden = 0;
    sc::ladder_host ladder{};
    uint32_t tiles_per_run = 1, partial_slots = 0, quantities = 0, backward_split = 1, spec_code = 0;
    bool fused = false;
    uint64_t gradients = 0, gradients_bytes = 0; // the gradient cube, or the fused kernel's patch scratch
    uint64_t transposed = 0, query_gradient = 0, partials = 0, accumulators = 0, status = 0;
    uint64_t budget_ns = 0;
    int multiprocessors = 0;

    bool transpose_candidates = true; // false: the backward kernel reads the block as it lies (MN-major operand)

    // Overlap of one block's backward GEMM with the next block's forward kernel. The two kernels want different parts
    // of the chip (the forward is bound by its epilogue arithmetic, the backward by memory), so inside a step of
    // several blocks the backward of block b runs on a second stream on `backward_multiprocessors` multiprocessors while
    // the forward of block b+1, launched first and with its persistent grid cut by that many, runs on the rest. It takes
    // a second gradient cube (`gradients_alt`); a block's candidates must stay in place until the block after next is
    // scored. The last backward of a step runs on the caller's stream in `join`.
    bool overlap = false;
    int backward_multiprocessors = 0;
    uint64_t gradients_alt = 0;
    // `front` (highest priority) carries the forward kernels and `side` (lowest) the overlapped backward kernels: when
    // both have blocks waiting for a multiprocessor, the forward's are placed first, whichever kernel started first.
    cudaStream_t side = nullptr, front = nullptr;
    cudaEvent_t forward_done[2] = {nullptr, nullptr}, backward_done[2] = {nullptr, nullptr};
    cudaEvent_t forked[2] = {nullptr, nullptr}, rejoined[2] = {nullptr, nullptr};
    uint32_t scored = 0;
    bool pending = false;
    uint32_t pending_slot = 0;
    sc::backward_arguments pending_backward{};

    loss_plan() = default;
    loss_plan(loss_plan const&) = delete; // owns streams and events
    loss_plan& operator=(loss_plan const&) = delete;
    ~loss_plan() {
        for (cudaEvent_t event : {forward_done[0], forward_done[1], backward_done[0], backward_done[1], forked[0], forked[1],
                                  rejoined[0], rejoined[1]})
            if (event) cudaEventDestroy(event);
        if (side) cudaStreamDestroy(side);
        if (front) cudaStreamDestroy(front);
    }

    void enable_overlap(uint64_t second_cube, int reserved) {
        if (fused) throw std::runtime_error("LossPlan: the fused kernel has no separate backward to overlap");
        if (reserved < 1 || reserved >= multiprocessors)
            throw std::runtime_error("LossPlan: the backward's share of the multiprocessors must lie in [1, all)");
        if (!second_cube) throw std::runtime_error("LossPlan: overlap needs a second gradient cube");
        if (!side) {
            int least = 0, greatest = 0;
            runtime_check(cudaDeviceGetStreamPriorityRange(&least, &greatest), "cudaDeviceGetStreamPriorityRange");
            runtime_check(cudaStreamCreateWithPriority(&side, cudaStreamNonBlocking, least), "cudaStreamCreateWithPriority");
            runtime_check(cudaStreamCreateWithPriority(&front, cudaStreamNonBlocking, greatest), "cudaStreamCreateWithPriority");
            for (cudaEvent_t* event : {&forward_done[0], &forward_done[1], &backward_done[0], &backward_done[1], &forked[0],
                                       &forked[1], &rejoined[0], &rejoined[1]})
                runtime_check(cudaEventCreateWithFlags(event, cudaEventDisableTiming), "cudaEventCreateWithFlags");
        }
        gradients_alt = second_cube, backward_multiprocessors = reserved, overlap = true;
    }

    // Starts a step: no backward is in flight (join() ended the last one).
    void begin_step() {
        if (pending) throw std::runtime_error("LossPlan: begin_step with a backward still pending (join() was not called)");
        scored = 0;
    }

    void launch_pending_on_side() {
        runtime_check(cudaStreamWaitEvent(side, forward_done[pending_slot], 0), "cudaStreamWaitEvent");
        sc::launch_backward(pending_backward, side);
        runtime_check(cudaEventRecord(backward_done[pending_slot], side), "cudaEventRecord");
        pending = false;
    }

    // Ends a step on `stream`: everything the side stream still runs is waited for, and the last block's backward runs
    // here with the whole chip.
    void join(uint64_t stream_handle) {
        cudaStream_t const stream = stream_of(stream_handle);
        if (overlap && scored >= 2) {
            // the backward of the block before the last one (and, through stream order, all earlier ones)
            runtime_check(cudaStreamWaitEvent(stream, backward_done[(scored & 1u)], 0), "cudaStreamWaitEvent");
        }
        if (pending) {
            sc::launch_backward(pending_backward, stream);
            pending = false;
        }
        scored = 0;
    }

    void score(uint64_t queries, uint64_t candidates, uint64_t q_inv, uint64_t c_inv, uint64_t c_tile_max, uint64_t query_base,
               uint64_t candidate_base, float beta, float bias, double live, uint64_t scalars, uint64_t pull_src0,
               uint64_t pull_dst0, uint64_t pull_bytes0, uint64_t pull_src1, uint64_t pull_dst1, uint64_t pull_bytes1,
               uint64_t stream_handle) {
        cudaStream_t const stream = stream_of(stream_handle);
        bool const transposing = fused || transpose_candidates || hidden < 64;
        bool const overlapping = overlap && !transposing;
        uint32_t const slot = overlapping ? scored & 1u : 0u;
        uint64_t const cube = slot ? gradients_alt : gradients;
        // this cube was last read by the backward of the block before the previous one
        if (overlapping && scored >= 2) runtime_check(cudaStreamWaitEvent(stream, backward_done[slot], 0), "cudaStreamWaitEvent");
        if (transposing) sc::launch_transpose(pointer<void>(candidates), pointer<void>(transposed), rows_c, hidden, stream);
        sc::forward_arguments a{};
        a.queries_bf16 = pointer<void>(queries), a.candidates_bf16 = pointer<void>(candidates);
        a.query_inverse_norms = pointer<float>(q_inv), a.candidate_inverse_norms = pointer<float>(c_inv);
        a.candidate_tile_max = pointer<float>(c_tile_max);
        a.gradient_cube_bf16 = pointer<void>(cube), a.partials = pointer<float>(partials);
        a.status = pointer<uint32_t>(status);
        a.rows_q = rows_q, a.rows_c = rows_c, a.hidden = hidden, a.ladder = ladder;
        a.tiles_per_run = tiles_per_run, a.beta = beta, a.bias = bias, a.weight = static_cast<float>(1.0 / live);
        a.scalars = pointer<float>(scalars);
        a.query_base = query_base, a.candidate_base = candidate_base, a.spec_code = spec_code, a.budget_ns = budget_ns;
        a.pull.src[0] = pointer<void>(pull_src0), a.pull.dst[0] = pointer<void>(pull_dst0), a.pull.bytes[0] = pull_bytes0;
        a.pull.src[1] = pointer<void>(pull_src1), a.pull.dst[1] = pointer<void>(pull_dst1), a.pull.bytes[1] = pull_bytes1;
        // a forward that has the previous block's backward beside it leaves that kernel its multiprocessors
        a.multiprocessors = overlapping && pending ? multiprocessors - backward_multiprocessors : multiprocessors;
        a.fused = fused, a.fused_scratch_bf16 = pointer<void>(cube), a.fused_scratch_bytes = gradients_bytes;
        a.transposed_candidates = pointer<void>(transposed), a.query_gradient = pointer<float>(query_gradient);
        a.gradient_scale = static_cast<float>(2.0 / live);
        if (overlapping && pending) {
            runtime_check(cudaEventRecord(forked[slot], stream), "cudaEventRecord");
            runtime_check(cudaStreamWaitEvent(front, forked[slot], 0), "cudaStreamWaitEvent");
            sc::launch_forward(a, front);
            // the previous block's backward goes out once this block's forward is in its queue
            launch_pending_on_side();
            runtime_check(cudaEventRecord(rejoined[slot], front), "cudaEventRecord");
            runtime_check(cudaStreamWaitEvent(stream, rejoined[slot], 0), "cudaStreamWaitEvent");
        } else sc::launch_forward(a, stream);
        sc::launch_fold_partials(pointer<float>(partials), pointer<float>(accumulators), rows_q, partial_slots, quantities, stream);
        if (!fused) {
            sc::backward_arguments b{};
            b.gradient_cube_bf16 = pointer<void>(cube);
            b.transposed_candidates = transposing ? pointer<void>(transposed) : nullptr;
            b.candidates_row_major = transposing ? nullptr : pointer<void>(candidates);
            b.query_gradient = pointer<float>(query_gradient), b.status = pointer<uint32_t>(status);
            b.rows_q = rows_q, b.rows_c = rows_c, b.hidden = hidden, b.ladder = ladder, b.split = backward_split;
            b.scale = static_cast<float>(2.0 / live), b.budget_ns = budget_ns;
            if (!overlapping) sc::launch_backward(b, stream);
            else {
                runtime_check(cudaEventRecord(forward_done[slot], stream), "cudaEventRecord");
                pending_backward = b, pending_slot = slot, pending = true;
            }
        }
        ++scored;
    }
};

torch::Tensor tensor_from_pointer(uint64_t address, std::vector<int64_t> sizes, std::string const& dtype, int device) {
    torch::ScalarType type;
    if (dtype == "float32") type = torch::kFloat32;
    else if (dtype == "bfloat16") type = torch::kBFloat16;
    else if (dtype == "uint8") type = torch::kUInt8;
    else if (dtype == "int32") type = torch::kInt32;
    else if (dtype == "int64") type = torch::kInt64;
    else throw std::runtime_error("tensor_from_pointer: unsupported dtype " + dtype);
    auto options = torch::TensorOptions().dtype(type).device(torch::kCUDA, device);
    return torch::from_blob(pointer<void>(address), sizes, [](void*) {}, options);
}

} // namespace

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
    m.doc() = "sm_100a kernels and the symmetric-memory domain of scalingcontrasts_b200";
    m.def("launch_count", &sc::launch_count);
    m.def("tensor_from_pointer", &tensor_from_pointer);
    m.attr("CONTROL_BYTES") = 256;
    m.attr("STATUS_OFFSET") = control_status;
    m.attr("ROUND_OFFSET") = control_round;
    m.attr("FLAG_OFFSET") = control_flag;
    m.attr("FINISHED_OFFSET") = control_finished;

    py::class_<sc::native_domain, std::shared_ptr<sc::native_domain>>(m, "NativeDomain")
        .def(py::init<int, int, int, size_t, bool>())
        .def_static("multicast_supported", &sc::native_domain::multicast_supported)
        .def("export_replica", &sc::native_domain::export_replica)
        .def("import_replica", &sc::native_domain::import_replica)
        .def("create_multicast", &sc::native_domain::create_multicast)
        .def("import_multicast", &sc::native_domain::import_multicast)
        .def("add_device", &sc::native_domain::add_device)
        .def("map_replicas", &sc::native_domain::map_replicas)
        .def("bind_multicast", &sc::native_domain::bind_multicast)
        .def("zero_own", &sc::native_domain::zero_own)
        .def("close", &sc::native_domain::close)
        .def("replica", &sc::native_domain::replica)
        .def("multicast", &sc::native_domain::multicast)
        .def("stride", &sc::native_domain::stride)
        .def("has_multicast", &sc::native_domain::has_multicast)
        .def("members", &sc::native_domain::members)
        .def("member", &sc::native_domain::member);

    py::class_<control_handle, std::shared_ptr<control_handle>>(m, "Control")
        .def("set_budget_ns", [](control_handle& c, uint64_t ns) { c.view.budget_ns = ns; })
        .def("budget_ns", [](control_handle const& c) { return c.view.budget_ns; })
        .def("uses_multicast", [](control_handle const& c) { return c.view.multicast_flag != nullptr; });
    m.def("make_control", &make_control);
    m.def("preload_kernels", []() {
        sc::preload_collective_kernels();
        sc::preload_loss_kernels();
    });

    m.def("barrier", [](control_handle const& c, uint64_t stream) { sc::launch_barrier(c.view, stream_of(stream)); });
    m.def("expect_arrivals", [](control_handle const& c, uint32_t arrivals, uint64_t stream) {
        sc::launch_expect_arrivals(c.view, arrivals, stream_of(stream));
    });
    m.def("all_reduce", [](control_handle const& c, uint64_t byte_offset, uint64_t scalars, int type, float scale, int sms,
                           uint64_t stream) {
        auto const kind = static_cast<sc::payload_type>(type);
        uint64_t const width = kind == sc::payload_type::f32 ? 4 : 2;
        if (byte_offset % 16) throw std::runtime_error("all_reduce: the payload must start on a 16-byte boundary");
        // Offsets are applied to the base pointers so that `first` stays zero and element indices stay small.
        std::vector<void*> replicas;
        for (void* base : c.replicas) replicas.push_back(static_cast<char*>(base) + byte_offset);
        void* multicast = c.multicast_base ? pointer<void>(c.multicast_base + byte_offset) : nullptr;
        (void)width;
        sc::launch_all_reduce(c.view, multicast, replicas.data(), 0, scalars, kind, scale, sms, stream_of(stream));
    });
    m.def("all_reduce_small", [](control_handle const& c, uint64_t byte_offset, uint64_t scalars, int type, float scale,
                                 uint64_t slots_offset, uint64_t slot_bytes, uint64_t stream) {
        if (byte_offset % 16 || slots_offset % 16) throw std::runtime_error("all_reduce_small: offsets must be multiples of 16");
        std::vector<void*> slot_replicas;
        for (void* base : c.replicas) slot_replicas.push_back(static_cast<char*>(base) + slots_offset);
        void* multicast = c.multicast_base ? pointer<void>(c.multicast_base + slots_offset) : nullptr;
        sc::launch_all_reduce_small(c.view, pointer<void>(c.own_base + byte_offset), multicast, slot_replicas.data(),
                                    pointer<void>(c.own_base + slots_offset), scalars, static_cast<sc::payload_type>(type), scale,
                                    slot_bytes, stream_of(stream));
    });
    m.def("last_collective_path", &sc::last_collective_path);
    m.def("reduce_scatter", [](control_handle const& c, uint64_t byte_offset, uint64_t shard_scalars, int type, float scale,
                               uint64_t out_f32, int sms, uint64_t stream) {
        auto const kind = static_cast<sc::payload_type>(type);
        if (byte_offset % 16) throw std::runtime_error("reduce_scatter: the payload must start on a 16-byte boundary");
        std::vector<void*> replicas;
        for (void* base : c.replicas) replicas.push_back(static_cast<char*>(base) + byte_offset);
        void* multicast = c.multicast_base ? pointer<void>(c.multicast_base + byte_offset) : nullptr;
        sc::launch_reduce_scatter(c.view, multicast, replicas.data(), pointer<void>(c.own_base + byte_offset), 0, shard_scalars,
                                  kind, scale, pointer<float>(out_f32), sms, stream_of(stream));
    });

    m.def("prefix_norms", [](uint64_t rows, uint64_t copy, uint64_t inverse_norms, uint64_t tile_max, uint32_t row_count,
                             uint32_t hidden, std::vector<uint32_t> const& ends, uint64_t stream) {
        sc::launch_prefix_norms(pointer<void>(rows), pointer<void>(copy), pointer<float>(inverse_norms), pointer<float>(tile_max),
                                row_count, hidden, ladder_of(ends), stream_of(stream));
    });
    m.def("transpose", [](uint64_t rows, uint64_t out, uint32_t row_count, uint32_t hidden, uint64_t stream) {
        sc::launch_transpose(pointer<void>(rows), pointer<void>(out), row_count, hidden, stream_of(stream));
    });
    m.def("pull", [](uint64_t src0, uint64_t dst0, uint64_t bytes0, uint64_t src1, uint64_t dst1, uint64_t bytes1, int blocks,
                     uint64_t stream) {
        sc::launch_pull(pointer<void>(src0), pointer<void>(dst0), bytes0, pointer<void>(src1), pointer<void>(dst1), bytes1, blocks,
                        stream_of(stream));
    });
    m.def("fold_partials", [](uint64_t partials, uint64_t accumulators, uint32_t rows, uint32_t slots, uint32_t quantities,
                              uint64_t stream) {
        sc::launch_fold_partials(pointer<float>(partials), pointer<float>(accumulators), rows, slots, quantities, stream_of(stream));
    });
    m.def("finalize", [](uint64_t queries, uint64_t inverse_norms, uint64_t accumulators, uint64_t query_gradient, uint64_t out,
                         uint32_t rows, uint32_t hidden, std::vector<uint32_t> const& ends, uint64_t stream) {
        sc::launch_finalize(pointer<void>(queries), pointer<float>(inverse_norms), pointer<float>(accumulators),
                            pointer<float>(query_gradient), pointer<void>(out), rows, hidden, ladder_of(ends), stream_of(stream));
    });
    m.def("sum_summands", [](uint64_t accumulators, uint64_t summands, uint32_t rows, uint32_t prefixes, uint64_t stream) {
        sc::launch_sum_summands(pointer<float>(accumulators), pointer<float>(summands), rows, prefixes, stream_of(stream));
    });
    py::class_<loss_plan, std::shared_ptr<loss_plan>>(m, "LossPlan")
        .def(py::init([](uint32_t rows_q, uint32_t rows_c, uint32_t hidden, std::vector<uint32_t> const& ends,
                         uint32_t tiles_per_run, uint32_t partial_slots, uint32_t quantities, uint32_t backward_split,
                         uint32_t spec_code, bool fused, uint64_t gradients, uint64_t gradients_bytes, uint64_t transposed,
                         uint64_t query_gradient, uint64_t partials, uint64_t accumulators, uint64_t status,
                         uint64_t budget_ns, int multiprocessors) {
                 auto plan = std::make_shared<loss_plan>();
                 plan->rows_q = rows_q, plan->rows_c = rows_c, plan->hidden = hidden, plan->ladder = ladder_of(ends);
                 plan->tiles_per_run = tiles_per_run, plan->partial_slots = partial_slots, plan->quantities = quantities;
                 plan->backward_split = backward_split, plan->spec_code = spec_code, plan->fused = fused;
                 plan->gradients = gradients, plan->gradients_bytes = gradients_bytes, plan->transposed = transposed;
                 plan->query_gradient = query_gradient, plan->partials = partials, plan->accumulators = accumulators;
                 plan->status = status, plan->budget_ns = budget_ns, plan->multiprocessors = multiprocessors;
                 return plan;
             }),
             py::arg("rows_q"), py::arg("rows_c"), py::arg("hidden"), py::arg("ends"), py::arg("tiles_per_run"),
             py::arg("partial_slots"), py::arg("quantities"), py::arg("backward_split"), py::arg("spec_code"), py::arg("fused"),
             py::arg("gradients"), py::arg("gradients_bytes"), py::arg("transposed"), py::arg("query_gradient"),
             py::arg("partials"), py::arg("accumulators"), py::arg("status"), py::arg("budget_ns"), py::arg("multiprocessors"))
        .def_readwrite("transpose_candidates", &loss_plan::transpose_candidates)
        .def_readonly("overlap", &loss_plan::overlap)
        .def("enable_overlap", &loss_plan::enable_overlap, py::arg("second_cube"), py::arg("backward_multiprocessors"))
        .def("begin_step", &loss_plan::begin_step)
        .def("join", &loss_plan::join, py::arg("stream"))
        .def("score", &loss_plan::score);
    m.attr("BOUNDS_BUILD") = sc::bounds_build();
    m.def("bounds_records", []() {
        // the first out-of-range index each translation unit recorded (all zeros: none); ordinary builds never record
        std::vector<std::vector<uint32_t>> records(6, std::vector<uint32_t>(8, 0u));
        sc::bounds_record_tower(records[4].data());
        sc::bounds_record_optim(records[5].data());
        sc::bounds_record_small(records[0].data());
        sc::bounds_record_forward(records[1].data());
        sc::bounds_record_backward(records[2].data());
        sc::bounds_record_collectives(records[3].data());
        return records;
    });
    m.def("backward_plan", [](uint32_t rows_q, std::vector<uint32_t> const& ends, uint32_t split, int multiprocessors) {
        uint32_t ctas = 0;
        auto const tiles = sc::backward_plan(rows_q, ladder_of(ends), split, multiprocessors, &ctas);
        return py::make_tuple(tiles, ctas);
    }, py::arg("rows_q"), py::arg("ends"), py::arg("split") = 1, py::arg("multiprocessors") = 148);
    m.def("adamw_step",
          [](std::vector<std::tuple<uint64_t, uint64_t, uint64_t, uint64_t, uint64_t, bool>> const& entries, float lr,
             float beta1, float beta2, float eps, float weight_decay, uint64_t step, uint64_t stream) {
              // one entry per tensor: (parameter, gradient, first moment, second moment, element count, is bfloat16)
              std::vector<sc::adamw_tensor> tensors;
              for (auto const& [param, grad, exp_avg, exp_avg_sq, count, is_bf16] : entries)
                  tensors.push_back(sc::adamw_tensor{pointer<void>(param), pointer<void>(grad), pointer<float>(exp_avg),
                                                     pointer<float>(exp_avg_sq), static_cast<size_t>(count), is_bf16 ? 1u : 0u, 0u});
              sc::launch_adamw(tensors.data(), static_cast<uint32_t>(tensors.size()), lr, beta1, beta2, eps, weight_decay, step,
                               stream_of(stream));
          },
          py::arg("entries"), py::arg("lr"), py::arg("beta1"), py::arg("beta2"), py::arg("eps"), py::arg("weight_decay"),
          py::arg("step"), py::arg("stream"));
    m.def("note_launches", [](uint64_t count) { sc::note_launch(count); });
    m.def("forward_partial_slots", &sc::forward_partial_slots);
    m.def("forward_quantities", &sc::forward_quantities);
    m.def("forward_choose_tiles_per_run", &sc::forward_choose_tiles_per_run);
    m.def("forward_fused_supported", &sc::forward_fused_supported);
    m.def("forward_choose_tiles_per_run_fused", &sc::forward_choose_tiles_per_run_fused);
    m.def("forward_fused_scratch_bytes", &sc::forward_fused_scratch_bytes);
    m.def("forward",
          [](uint64_t queries, uint64_t candidates, uint64_t q_inv, uint64_t c_inv, uint64_t c_tile_max, uint64_t cube,
             uint64_t partials, uint64_t status, uint32_t rows_q, uint32_t rows_c, uint32_t hidden,
             std::vector<uint32_t> const& ends, uint32_t tiles_per_run, float beta, float bias, float weight, uint64_t scalars,
             uint64_t query_base,
             uint64_t candidate_base, uint32_t spec_code, uint64_t budget_ns, uint64_t pull_src0, uint64_t pull_dst0,
             uint64_t pull_bytes0, uint64_t pull_src1, uint64_t pull_dst1, uint64_t pull_bytes1, int sms, uint64_t stream,
             uint64_t trace, bool fused, uint64_t fused_scratch, uint64_t fused_scratch_bytes, uint64_t transposed,
             uint64_t query_gradient, float gradient_scale) {
              sc::forward_arguments a{};
              a.queries_bf16 = pointer<void>(queries), a.candidates_bf16 = pointer<void>(candidates);
              a.query_inverse_norms = pointer<float>(q_inv), a.candidate_inverse_norms = pointer<float>(c_inv);
              a.candidate_tile_max = pointer<float>(c_tile_max);
              a.gradient_cube_bf16 = pointer<void>(cube), a.partials = pointer<float>(partials);
              a.status = pointer<uint32_t>(status);
              a.rows_q = rows_q, a.rows_c = rows_c, a.hidden = hidden, a.ladder = ladder_of(ends);
              a.tiles_per_run = tiles_per_run, a.beta = beta, a.bias = bias, a.weight = weight;
              a.scalars = pointer<float>(scalars);
              a.query_base = query_base, a.candidate_base = candidate_base, a.spec_code = spec_code, a.budget_ns = budget_ns;
              a.pull.src[0] = pointer<void>(pull_src0), a.pull.dst[0] = pointer<void>(pull_dst0), a.pull.bytes[0] = pull_bytes0;
              a.pull.src[1] = pointer<void>(pull_src1), a.pull.dst[1] = pointer<void>(pull_dst1), a.pull.bytes[1] = pull_bytes1;
              a.multiprocessors = sms;
              a.trace = pointer<unsigned long long>(trace);
              a.fused = fused, a.fused_scratch_bf16 = pointer<void>(fused_scratch), a.fused_scratch_bytes = fused_scratch_bytes;
              a.transposed_candidates = pointer<void>(transposed), a.query_gradient = pointer<float>(query_gradient);
              a.gradient_scale = gradient_scale;
              sc::launch_forward(a, stream_of(stream));
          },
          py::arg("queries"), py::arg("candidates"), py::arg("q_inv"), py::arg("c_inv"), py::arg("c_tile_max"), py::arg("cube"),
          py::arg("partials"), py::arg("status"), py::arg("rows_q"), py::arg("rows_c"), py::arg("hidden"), py::arg("ends"),
          py::arg("tiles_per_run"), py::arg("beta"), py::arg("bias"), py::arg("weight"), py::arg("scalars"), py::arg("query_base"),
          py::arg("candidate_base"), py::arg("spec_code"), py::arg("budget_ns"), py::arg("pull_src0"), py::arg("pull_dst0"),
          py::arg("pull_bytes0"), py::arg("pull_src1"), py::arg("pull_dst1"), py::arg("pull_bytes1"), py::arg("sms"),
          py::arg("stream"), py::arg("trace") = 0, py::arg("fused") = false, py::arg("fused_scratch") = 0,
          py::arg("fused_scratch_bytes") = 0, py::arg("transposed") = 0, py::arg("query_gradient") = 0,
          py::arg("gradient_scale") = 0.0f);
    m.def("backward", [](uint64_t cube, uint64_t transposed, uint64_t query_gradient, uint64_t status, uint32_t rows_q,
                         uint32_t rows_c, uint32_t hidden, std::vector<uint32_t> const& ends, uint32_t split, float scale,
                         uint64_t budget_ns, uint64_t stream, uint64_t row_major) {
        sc::backward_arguments a{};
        a.gradient_cube_bf16 = pointer<void>(cube), a.transposed_candidates = pointer<void>(transposed);
        a.candidates_row_major = pointer<void>(row_major);
        a.query_gradient = pointer<float>(query_gradient), a.status = pointer<uint32_t>(status);
        a.rows_q = rows_q, a.rows_c = rows_c, a.hidden = hidden, a.ladder = ladder_of(ends), a.split = split, a.scale = scale;
        a.budget_ns = budget_ns;
        sc::launch_backward(a, stream_of(stream));
    }, py::arg("cube"), py::arg("transposed"), py::arg("query_gradient"), py::arg("status"), py::arg("rows_q"), py::arg("rows_c"),
       py::arg("hidden"), py::arg("ends"), py::arg("split"), py::arg("scale"), py::arg("budget_ns"), py::arg("stream"),
       py::arg("row_major") = 0);

    m.def("tower_partial_blocks", &sc::tower_partial_blocks);
    m.def("gelu_forward", [](uint64_t z, uint64_t h, uint64_t scalars, int sms, uint64_t stream) {
        sc::launch_gelu_forward(pointer<void>(z), pointer<void>(h), scalars, sms, stream_of(stream));
    });
    m.def("gelu_backward_bias", [](uint64_t upstream, uint64_t z, uint64_t dz, uint64_t partials, uint64_t bias_grad, uint32_t rows,
                                   uint32_t columns, uint64_t stream) {
        sc::launch_gelu_backward_bias(pointer<void>(upstream), pointer<void>(z), pointer<void>(dz), pointer<float>(partials),
                                      pointer<void>(bias_grad), rows, columns, stream_of(stream));
    });
    m.def("column_sums", [](uint64_t matrix, uint64_t partials, uint64_t sums, uint32_t rows, uint32_t columns, uint64_t stream) {
        sc::launch_column_sums(pointer<void>(matrix), pointer<float>(partials), pointer<void>(sums), rows, columns, stream_of(stream));
    });

    m.def("keyed_embeddings", [](uint64_t rows, uint32_t row_count, uint32_t hidden, uint64_t salt, float scale, uint64_t stream) {
        sc::launch_keyed_embeddings(pointer<void>(rows), row_count, hidden, salt, scale, stream_of(stream));
    });
    m.def("keyed_integers", [](uint64_t out, uint64_t scalars, uint64_t first, uint32_t members, uint32_t member, uint64_t stream) {
        sc::launch_keyed_integers(pointer<float>(out), scalars, first, members, member, stream_of(stream));
    });
    m.def("keyed_fractions", [](uint64_t out, uint64_t scalars, uint64_t first, uint32_t members, uint32_t member, uint64_t stream) {
        sc::launch_keyed_fractions(pointer<float>(out), scalars, first, members, member, stream_of(stream));
    });
    m.def("count_wrong_sums", [](uint64_t values, uint64_t scalars, uint64_t first, uint32_t members, uint64_t counter,
                                 uint64_t stream) {
        sc::launch_count_wrong_sums(pointer<float>(values), scalars, first, members, pointer<unsigned long long>(counter),
                                    stream_of(stream));
    });
    m.def("count_differences", [](uint64_t values, uint64_t expected, uint64_t scalars, uint64_t counter, uint64_t stream) {
        sc::launch_count_differences(pointer<float>(values), pointer<float>(expected), scalars,
                                     pointer<unsigned long long>(counter), stream_of(stream));
    });
    m.def("scale_cast", [](uint64_t src, uint64_t dst, uint64_t scalars, float scale, uint64_t stream) {
        sc::launch_scale_cast(pointer<float>(src), pointer<void>(dst), scalars, scale, stream_of(stream));
    });

    py::class_<sc::loopback_rail, std::shared_ptr<sc::loopback_rail>>(m, "LoopbackRail")
        .def(py::init<int, uint64_t, uint64_t, uint64_t, int, int, std::string const&, uint32_t>())
        .def("local_endpoint",
             [](sc::loopback_rail const& rail) {
                 return py::bytes(reinterpret_cast<char const*>(&rail.local()), sizeof(sc::rail_endpoint));
             })
        .def("connect",
             [](sc::loopback_rail& rail, std::string const& endpoint) {
                 if (endpoint.size() != sizeof(sc::rail_endpoint)) throw std::runtime_error("rail: malformed endpoint record");
                 sc::rail_endpoint remote;
                 std::memcpy(&remote, endpoint.data(), sizeof(remote));
                 rail.connect(remote);
             })
        .def("post_embeddings", &sc::loopback_rail::post_embeddings)
        .def("post_summands",
             [](sc::loopback_rail& rail, int row, std::vector<float> const& values) {
                 rail.post_summands(row, values.data(), static_cast<int>(values.size()));
             })
        .def("await_landed", &sc::loopback_rail::await_landed, py::call_guard<py::gil_scoped_release>())
        .def("read_summands",
             [](sc::loopback_rail const& rail, int row, int count) {
                 std::vector<float> out(static_cast<size_t>(count));
                 rail.read_summands(row, out.data(), count);
                 return out;
             })
        .def("inject_completion_error", &sc::loopback_rail::inject_completion_error)
        .def("drain", &sc::loopback_rail::drain)
        .def("close", &sc::loopback_rail::close)
        .def("posted", &sc::loopback_rail::posted)
        .def("consumed", &sc::loopback_rail::consumed);
    m.attr("ENDPOINT_BYTES") = sizeof(sc::rail_endpoint);

    m.def("oracle_loops", [](torch::Tensor world, std::vector<uint32_t> const& ends, double beta, double bias, uint32_t spec_code) {
        auto w = world.to(torch::kFloat64).contiguous().cpu();
        auto gradient = torch::zeros_like(w);
        auto out = torch::zeros({12}, torch::kFloat64);
        sc::oracle_loops_f64(w.data_ptr<double>(), w.size(0), w.size(1), ladder_of(ends), beta, bias, spec_code,
                             gradient.data_ptr<double>(), out.data_ptr<double>());
        return std::make_tuple(gradient, out);
    });
}
