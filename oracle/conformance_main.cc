// Conformance driver: the REAL Cellerator operation core (register_candidate, prepare_candidate,
// run_prepared_operation with validate_launch_bindings) driving the cellerator_b200 candidates.
//
// TEST INFRASTRUCTURE.  Built only where the Cellerator tree is available (oracle/Makefile target
// `conformance`): it compiles the reference's operation_core.cc / referee.cc / operation.cc /
// operation_signature.cc in place, cellerator_b200/host/b200_candidates.cc against the reference
// headers, and links libcellerator_b200.so.  The binary lands in oracle/_ref/ and travels to the
// GPU box with the tree.  Without a device it checks the host half of the seam (registration,
// capability query, policy rejections, prepare failing loudly); with a B200 it prepares and runs
// the forward, transpose and Blocked-ELL candidates through run_prepared_operation and compares
// the results with the reference's own double-precision referee.
#include "../cellerator_b200/host/b200_candidates.hh"

#include <Cellerator/compute/math/referee.hh>
#include <Cellerator/types.cuh>

#include <cuda_runtime_api.h>

#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <random>
#include <vector>

namespace core = ::cellerator::compute::math::core;
namespace cm = ::cellerator::compute::math;
namespace ex = ::cellerator::execution;
namespace host = ::cellerator_b200::host;

static int g_failures = 0;
#define CHECK(cond, name)                                                        \
    do {                                                                         \
        if (cond) std::printf("PASS %s\n", name);                                \
        else { std::printf("FAIL %s (%s:%d)\n", name, __FILE__, __LINE__); ++g_failures; } \
    } while (0)

template<typename Tag> static ex::identity_handle<Tag> handle(std::uint32_t slot) { return {slot, 1u}; }
static ex::axis_identity axis(std::uint32_t base) {
    return {handle<ex::domain_tag>(base), handle<ex::order_tag>(base + 1), handle<ex::geometry_tag>(base + 2),
            handle<ex::partition_tag>(7u)};
}

static core::numeric_policy policy_u8(ex::numeric_type dense) {
    core::numeric_policy n;
    n.sparse_storage = ex::numeric_type::u8;
    n.dense_storage = dense;
    n.output_storage = ex::numeric_type::f32;
    n.multiply = ex::numeric_type::f32;
    n.accumulation = ex::numeric_type::f32;
    n.scalar = ex::numeric_type::f32;
    n.quantization = core::quantization_granularity::value_plane;
    return n;
}

template<typename T> static T *to_device(const std::vector<T> &v) {
    T *d = nullptr;
    if (cudaMalloc(reinterpret_cast<void **>(&d), (v.size() + 1) * sizeof(T)) != cudaSuccess) std::abort();
    cudaMemcpy(d, v.data(), v.size() * sizeof(T), cudaMemcpyHostToDevice);
    return d;
}

struct problem_ids {
    core::operation_problem problem;
    core::structure_set_key structures;
    core::projection_key projection;
};

static problem_ids make_ids(std::uint32_t salt, core::projection_kind kind, std::uint64_t work) {
    problem_ids ids{};
    ids.problem.kind = core::operation_kind::sparse_dense_multiply;
    ids.problem.operation = {0x5eedull + salt, 1ull};
    ids.problem.input_count = 2u;
    ids.problem.output_count = 1u;
    ids.problem.logical_work_items = work;
    ids.structures.count = 1u;
    ids.structures.structures[0].persistent = {0x57ull + salt, 2ull};
    ids.structures.structures[0].runtime = handle<ex::structure_tag>(10u + salt);
    ids.structures.structures[0].epoch = {3u};
    ids.projection.persistent = {0x9aull + salt, 4ull};
    ids.projection.runtime = handle<ex::projection_tag>(20u + salt);
    ids.projection.kind = kind;
    ids.projection.schema_version = 1u;
    return ids;
}

// plan_end_to_end (src/planner/end_to_end_planner.cc:268-518) over one planner_candidate per (operation candidate,
// schedule) at the benchmark configuration's shape: the reference's own rejection rules and analytical ranking
// decide.  No device is touched: the records come from host arithmetic on the shape.
static void planner_leg(const core::candidate_registry &registry) {
    namespace pl = ::cellerator::planner;
    const core::operation_candidate *fwd = core::find_candidate(registry, host::quantized_csr_forward_candidate().identity);
    const core::operation_candidate *tr = core::find_candidate(registry, host::quantized_csr_transpose_candidate().identity);
    const core::operation_candidate *ord = core::find_candidate(registry, host::quantized_csr_transpose_ordered_candidate().identity);
    CHECK(fwd != nullptr && tr != nullptr && ord != nullptr, "planner: the candidates are registered");
    if (fwd == nullptr || tr == nullptr || ord == nullptr) return;
    // 1,000,000 cells x 33,538 genes, 1.8e9 stored entries, N = 64: the matrix is described, not allocated
    cb200_qcsr dm{};
    dm.version = CB200_ABI_VERSION; dm.size = sizeof dm; dm.rows = 1000000; dm.cols = 33538; dm.nnz = 1797264673ll; dm.bits = 8;
    dm.policy = CB200_DECODE_PER_GENE_AFFINE;
    const auto request_for = [&](const problem_ids &ids, const pl::planner_candidate *candidates, std::uint32_t count) {
        pl::planner_request r{};
        r.problem = ids.problem;
        r.keys.problem.identity = ids.problem.operation;
        pl::make_persistent_structure_set_key(ids.structures, &r.keys.structures);
        r.keys.geometry = {{1u, 1u}, {2u, 1u}, {3u, 1u}, {4u, 1u}, {5u, 1u}, {6u, 1u}};
        r.keys.device = {0x10deu, 10u, 0u, 1u};
        r.keys.build = {12090u, 1u, 580u, 2u};
        r.keys.policy.structure_reuse = 1000u;
        r.keys.policy.projection_reuse = 1000u;
        r.candidates = candidates;
        r.candidate_count = count;
        r.current_evidence_revision = 1u;
        return r;
    };
    const auto variant_of = [](const pl::planner_result &res) { return res.selected != nullptr ? res.selected->projection.variant : 0xffffffffu; };

    // ---- forward, bf16 W, bf16 products allowed, the matrix at hand
    problem_ids f = make_ids(30u, core::projection_kind::csr, static_cast<std::uint64_t>(dm.nnz));
    host::projection_catalog_entry fs{};
    fs.projection = f.projection.runtime; fs.projection_kind = CB200_PROJECTION_CSR;
    fs.m = dm.rows; fs.k = dm.cols; fs.n = 64; fs.nnz = dm.nnz; fs.bits = 8; fs.dense_dtype = CB200_DTYPE_BF16; fs.device_matrix = &dm;
    const pl::planner_candidate forward[3] = {
        host::make_schedule_candidate(*fwd, f.projection, fs, host::schedule_gene_tiled, CB200_DTYPE_BF16, 6553.9),
        host::make_schedule_candidate(*fwd, f.projection, fs, host::schedule_tensor_blocked, CB200_DTYPE_BF16, 6553.9),
        host::make_schedule_candidate(*fwd, f.projection, fs, host::schedule_warp_per_row, CB200_DTYPE_BF16, 6553.9)};
    CHECK(forward[1].analytical.persistent_bytes > 7000000000ull && forward[1].analytical.persistent_bytes < 7400000000ull &&
              forward[0].analytical.persistent_bytes == 0u,
          "planner: the window-blocked schedule declares its persistent copy (one word per entry), the exact ones none");
    pl::planner_result res{};
    pl::planner_request req = request_for(f, forward, 3u);
    pl::planner_status st = pl::plan_end_to_end(req, &res);
    CHECK(static_cast<bool>(st) && res.legal_count == 3u && res.source == pl::selection_source::analytical && res.tuning_skipped &&
              variant_of(res) == host::schedule_tensor_blocked,
          "planner: the tensor-core schedule over the window-blocked copy wins the forward projection on analytical cost");
    if (!st) std::printf("  message: %s\n", st.message);
    // the prepare of the copy is amortised: a one-shot request pays all of it, and the exact kernel wins
    req.keys.policy.structure_reuse = req.keys.policy.projection_reuse = 1u;
    st = pl::plan_end_to_end(req, &res);
    CHECK(static_cast<bool>(st) && variant_of(res) == host::schedule_gene_tiled, "planner: a one-shot request does not pay for the copy");
    req.keys.policy.structure_reuse = req.keys.policy.projection_reuse = 1000u;
    // persistent-memory limit below the copy: rejected as persistent_memory, the exact gene-tiled kernel is next
    req.policy.maximum_persistent_bytes = 1ull << 30;
    st = pl::plan_end_to_end(req, &res);
    CHECK(static_cast<bool>(st) && res.legal_count == 2u && res.diagnostics[1].rejection == pl::candidate_rejection::persistent_memory &&
              variant_of(res) == host::schedule_gene_tiled,
          "planner: the persistent-memory limit rejects the window-blocked copy and the gene-tiled kernel is selected");
    // an empirical pass: the measurement hook confirms the analytical order with measured times
    req.policy.maximum_persistent_bytes = 0u;
    struct measured_times { int calls; };
    measured_times ctx{0};
    req.measurement.context = &ctx;
    req.measurement.measure = [](void *c, const pl::planner_candidate &cand, pl::measured_candidate *m) noexcept -> bool {
        ++static_cast<measured_times *>(c)->calls;
        m->correct = true;
        m->sample_count = 20u;
        m->spread_percent = 0.3;
        m->phases = cand.analytical;
        // measured on B200, ms per launch: tensor_blocked 6.31, gene_tiled 20.3, warp_per_row 28.5
        m->phases.kernel_ns = cand.projection.variant == host::schedule_tensor_blocked ? 6.31e6
                              : cand.projection.variant == host::schedule_gene_tiled ? 20.3e6 : 28.5e6;
        return true;
    };
    st = pl::plan_end_to_end(req, &res);
    CHECK(static_cast<bool>(st) && res.source == pl::selection_source::empirical && ctx.calls == 3 && res.measurement_count == 3u &&
              variant_of(res) == host::schedule_tensor_blocked && res.confidence > 0.8,
          "planner: bounded tuning measures the shortlist and keeps the tensor-core schedule");

    // ---- transpose, fp32 G: the atomic-order schedules are not deterministic, the ordered gather is
    problem_ids t = make_ids(31u, core::projection_kind::transpose_or_backward, static_cast<std::uint64_t>(dm.nnz));
    host::projection_catalog_entry ts = fs;
    ts.projection = t.projection.runtime; ts.projection_kind = CB200_PROJECTION_TRANSPOSE; ts.dense_dtype = CB200_DTYPE_F32;
    const pl::planner_candidate transposes[3] = {
        host::make_schedule_candidate(*tr, t.projection, ts, host::schedule_vector_reductions, CB200_DTYPE_F32, 6553.9),
        host::make_schedule_candidate(*tr, t.projection, ts, host::schedule_tensor_blocked, CB200_DTYPE_F32, 6553.9),
        host::make_schedule_candidate(*ord, t.projection, ts, host::schedule_gene_gather, CB200_DTYPE_F32, 6553.9)};
    CHECK((transposes[0].flags & pl::planner_candidate_deterministic) == 0u && (transposes[2].flags & pl::planner_candidate_deterministic) != 0u,
          "planner: only the ordered transpose is flagged deterministic");
    CHECK(transposes[1].analytical.persistent_bytes > 14000000000ull && transposes[2].analytical.persistent_bytes > 8900000000ull,
          "planner: split-product words (8 B per entry) and the gene-major copy (5 B per entry) are declared");
    pl::planner_request treq = request_for(t, transposes, 3u);
    st = pl::plan_end_to_end(treq, &res);
    CHECK(static_cast<bool>(st) && res.legal_count == 3u && variant_of(res) == host::schedule_tensor_blocked,
          "planner: the split-product tensor schedule wins the transpose on analytical cost");
    treq.policy.deterministic = true;
    st = pl::plan_end_to_end(treq, &res);
    CHECK(static_cast<bool>(st) && res.legal_count == 1u && res.diagnostics[0].rejection == pl::candidate_rejection::nondeterministic &&
              res.diagnostics[1].rejection == pl::candidate_rejection::nondeterministic && variant_of(res) == host::schedule_gene_gather,
          "planner: a deterministic policy rejects the atomic-order transposes and selects the ordered gather");
    treq.policy.maximum_persistent_bytes = 1ull << 30; // ... which needs its gene-major copy
    st = pl::plan_end_to_end(treq, &res);
    CHECK(st.code == pl::planner_status_code::no_legal_candidate, "planner: deterministic and no room for the gene-major copy -> no legal candidate");
    // a record whose projection kind is not its operation's is malformed (end_to_end_planner.cc:81-96)
    pl::planner_candidate wrong = forward[0];
    wrong.projection.kind = core::projection_kind::transpose_or_backward;
    pl::planner_request wreq = request_for(f, &wrong, 1u);
    st = pl::plan_end_to_end(wreq, &res);
    CHECK(st.code == pl::planner_status_code::no_legal_candidate && res.diagnostics[0].rejection == pl::candidate_rejection::malformed,
          "planner: a record with the wrong projection kind is rejected as malformed");
}

int main(int argc, char **argv) {
    const bool host_only_requested = argc > 1 && std::strcmp(argv[1], "--host-only") == 0;
    int device_count = 0;
    const bool have_device = !host_only_requested && cudaGetDeviceCount(&device_count) == cudaSuccess && device_count > 0;
    std::printf("device: %s\n", have_device ? "present" : "none");

    // ---- registration and capability query (host only) ----------------------------------
    static core::candidate_registry registry;
    CHECK(static_cast<bool>(host::register_all(&registry)) && registry.size == 6u, "register six candidates");
    CHECK(core::register_candidate(&registry, host::quantized_csr_forward_candidate()).code ==
              core::operation_status_code::duplicate_candidate, "duplicate registration is rejected");
    const core::operation_candidate *fwd = core::find_candidate(registry, host::quantized_csr_forward_candidate().identity);
    const core::operation_candidate *tr = core::find_candidate(registry, host::quantized_csr_transpose_candidate().identity);
    const core::operation_candidate *bell = core::find_candidate(registry, host::quantized_blocked_ell_candidate().identity);
    CHECK(fwd != nullptr && tr != nullptr && bell != nullptr, "find_candidate by identity");
    CHECK(fwd->supports_numeric(policy_u8(ex::numeric_type::bf16)) && fwd->supports_numeric(policy_u8(ex::numeric_type::f32)),
          "forward supports bf16 and f32 W");
    CHECK(!fwd->supports_numeric(policy_u8(ex::numeric_type::f16)), "forward rejects f16 W");
    {
        core::numeric_policy n = policy_u8(ex::numeric_type::bf16);
        n.quantization = core::quantization_granularity::none;
        CHECK(!fwd->supports_numeric(n), "forward rejects an unquantized policy");
    }
    CHECK(tr->supports_numeric(policy_u8(ex::numeric_type::f32)) && !tr->supports_numeric(policy_u8(ex::numeric_type::bf16)),
          "transpose takes f32 G only");
    CHECK((tr->capability_flags & core::candidate_deterministic) == 0u, "transpose does not claim determinism");

    // ---- a small quantized CSR problem ---------------------------------------------------
    const std::int64_t M = 300, K = 1000, N = 64;
    std::mt19937 rng(7);
    std::vector<std::int64_t> row_ptr(M + 1, 0);
    std::vector<std::int32_t> col;
    for (std::int64_t r = 0; r < M; ++r) {
        std::vector<char> used(K, 0);
        const int want = static_cast<int>(rng() % 120);
        for (int i = 0; i < want; ++i) used[rng() % K] = 1;
        for (std::int64_t g = 0; g < K; ++g) if (used[g]) col.push_back(static_cast<std::int32_t>(g));
        row_ptr[r + 1] = static_cast<std::int64_t>(col.size());
    }
    const std::int64_t nnz = static_cast<std::int64_t>(col.size());
    std::vector<std::uint8_t> codes(nnz);
    for (auto &c : codes) c = static_cast<std::uint8_t>(rng() & 0xff);
    std::vector<float> scales(K), offsets(K), w(K * N), g(M * N);
    std::uniform_real_distribution<float> uni(0.01f, 0.05f), sym(-0.05f, 0.05f), one(-1.0f, 1.0f);
    for (auto &v : scales) v = uni(rng);
    for (auto &v : offsets) v = sym(rng);
    for (auto &v : w) v = sym(rng);
    for (auto &v : g) v = one(rng);

    const ex::axis_identity cells = axis(100u), genes = axis(200u), latent = axis(300u);
    problem_ids ids = make_ids(0u, core::projection_kind::csr, static_cast<std::uint64_t>(nnz));
    host::projection_catalog_entry shape{};
    shape.projection = ids.projection.runtime;
    shape.projection_kind = CB200_PROJECTION_CSR;
    shape.m = M; shape.k = K; shape.n = N; shape.nnz = nnz;
    shape.bits = 8; shape.dense_dtype = CB200_DTYPE_F32; shape.device = 0;
    shape.host_row_ptr = row_ptr.data();
    shape.cells = cells; shape.genes = genes; shape.latent = latent;
    CHECK(host::register_projection(shape), "projection catalog accepts the entry");

    // ---- policy rejections happen in prepare_candidate, before the backend is asked --------
    core::prepared_operation prepared{};
    {
        problem_ids t = make_ids(1u, core::projection_kind::transpose_or_backward, static_cast<std::uint64_t>(nnz));
        core::prepare_policy p;
        p.deterministic = true;
        CHECK(core::prepare_candidate(*tr, t.problem, t.structures, t.projection, policy_u8(ex::numeric_type::f32), p, &prepared).code ==
                  core::operation_status_code::capability_rejected, "deterministic policy rejects the transpose candidate");
        CHECK(core::prepare_candidate(*fwd, t.problem, t.structures, t.projection, policy_u8(ex::numeric_type::f32), {}, &prepared).code ==
                  core::operation_status_code::unsupported_projection, "projection kind mismatch is rejected");
        problem_ids unknown = make_ids(9u, core::projection_kind::csr, 10u);
        CHECK(core::prepare_candidate(*fwd, unknown.problem, unknown.structures, unknown.projection,
                                      policy_u8(ex::numeric_type::f32), {}, &prepared).code ==
                  core::operation_status_code::unsupported_projection, "unknown projection handle is rejected");
    }
    // ---- the reference's planner ranks the backend's schedules (host only) -----------------------------
    planner_leg(registry);

    if (!have_device) {
        const core::operation_status s = core::prepare_candidate(*fwd, ids.problem, ids.structures, ids.projection,
                                                                 policy_u8(ex::numeric_type::f32), {}, &prepared);
        CHECK(s.code == core::operation_status_code::preparation_failed && s.message != nullptr && s.message[0] != '\0',
              "prepare without a device fails loudly (no CPU fallback)");
        std::printf("%s: %d failure(s)\n", g_failures ? "FAILED" : "OK", g_failures);
        return g_failures ? 1 : 0;
    }

    // ---- device run through run_prepared_operation ----------------------------------------
    cudaSetDevice(0);
    std::int64_t *d_row_ptr = to_device(row_ptr);
    std::int32_t *d_col = to_device(col);
    std::uint8_t *d_codes = to_device(codes);
    float *d_scales = to_device(scales), *d_offsets = to_device(offsets), *d_w = to_device(w), *d_g = to_device(g);
    float *d_y = nullptr, *d_gt = nullptr;
    void *d_ws = nullptr;
    cudaMalloc(reinterpret_cast<void **>(&d_y), M * N * sizeof(float));
    cudaMalloc(reinterpret_cast<void **>(&d_gt), K * N * sizeof(float));
    cudaMalloc(&d_ws, 4096);
    cudaStream_t stream = nullptr;
    cudaStreamCreate(&stream);

    core::prepare_policy det;
    det.deterministic = true;
    core::operation_status st = core::prepare_candidate(*fwd, ids.problem, ids.structures, ids.projection,
                                                        policy_u8(ex::numeric_type::f32), det, &prepared);
    CHECK(static_cast<bool>(st), "prepare_candidate(forward, deterministic policy)");
    if (!st) std::printf("  message: %s\n", st.message);

    host::csr_projection_data proj{M, K, nnz, d_row_ptr, nullptr, d_col};
    const ex::device_location dev_loc{ex::residency_kind::device, {0, 0, 0}, 0, 0u};
    ex::relation_structure structure{ids.structures.structures[0].runtime, {3u}, cells, genes, {1u, 1u},
                                     static_cast<std::uint64_t>(nnz)};
    ex::value_plane plane{};
    plane.structure = structure.identity;
    plane.structure_epoch_value = {3u};
    plane.values = d_codes;
    plane.location = dev_loc;
    plane.numeric = {ex::numeric_type::u8, ex::numeric_type::f32, ex::numeric_type::f32, 0u};
    plane.quantization = {ex::quantization_kind::per_value_plane, ex::numeric_type::f32, ex::numeric_type::f32, 0u,
                          d_scales, d_offsets, static_cast<std::uint64_t>(K)};
    plane.layout = ex::value_layout_kind::logical_edge_order;
    plane.generation = {5u};
    plane.element_count = static_cast<std::uint64_t>(nnz);
    plane.value_bytes = static_cast<std::uint64_t>(nnz);
    ex::value_binding value{&plane, {5u}};

    auto dense_view = [&](void *data, const ex::axis_identity &a0, std::uint64_t rows) {
        ex::biological_operand_view v{};
        v.kind = ex::operand_kind::dense_tensor;
        v.storage.dense.data = data;
        v.storage.dense.location = dev_loc;
        v.storage.dense.value_type = ex::numeric_type::f32;
        v.storage.dense.rank = 2u;
        v.storage.dense.axes[0] = a0;
        v.storage.dense.axes[1] = latent;
        v.storage.dense.shape[0] = rows;
        v.storage.dense.shape[1] = static_cast<std::uint64_t>(N);
        v.storage.dense.stride[0] = N;
        v.storage.dense.stride[1] = 1;
        return v;
    };
    ex::biological_operand_view inputs[2]{};
    inputs[0].kind = ex::operand_kind::sparse_relation;
    inputs[0].storage.relation = {cells, genes, structure.identity, ids.projection.runtime, {3u}, &proj, sizeof proj,
                                  static_cast<std::uint64_t>(nnz), dev_loc};
    inputs[1] = dense_view(d_w, genes, static_cast<std::uint64_t>(K));
    ex::biological_operand_view outputs[1] = {dense_view(d_y, cells, static_cast<std::uint64_t>(M))};

    ex::launch_bindings launch{};
    launch.structures = &structure;
    launch.inputs = inputs;
    launch.outputs = outputs;
    launch.values = &value;
    launch.input_count = 2u;
    launch.output_count = 1u;
    launch.value_count = 1u;
    launch.structure_count = 1u;
    launch.stream = {stream, 0, 0u};
    launch.workspace = {d_ws, 4096u, dev_loc};

    st = core::run_prepared_operation(prepared, launch);
    CHECK(static_cast<bool>(st), "run_prepared_operation(forward)");
    if (!st) std::printf("  message: %s (binding %d)\n", st.message, static_cast<int>(st.binding));
    cudaStreamSynchronize(stream);
    std::vector<float> y(M * N);
    cudaMemcpy(y.data(), d_y, y.size() * sizeof(float), cudaMemcpyDeviceToHost);

    // the reference's own referee on the decoded values
    std::vector<float> decoded(nnz);
    for (std::int64_t i = 0; i < nnz; ++i) decoded[i] = static_cast<float>(codes[i]) * scales[col[i]] + offsets[col[i]];
    std::vector<cm::u64> offs(row_ptr.begin(), row_ptr.end());
    std::vector<cm::u32> ucol(col.begin(), col.end());
    auto referee = [&](bool transpose, const float *rhs, std::uint64_t rhs_rows, std::vector<double> *ref) {
        cm::spmm_request r;
        r.m = transpose ? K : M; r.k = transpose ? M : K; r.n = N; r.sparse_nnz = nnz;
        r.sparse_structure.identity_version = 1u; r.sparse_structure.value = 77u;
        r.transpose_sparse = transpose ? cm::transpose_kind::transpose : cm::transpose_kind::none;
        r.dense_rhs_leading_dimension = N; r.output_leading_dimension = N;
        r.sparse_storage_type_code = r.dense_storage_type_code = r.output_storage_type_code = ::cellerator::real::value_f32;
        r.compute_type_code = r.accumulation_type_code = ::cellerator::real::value_f64;
        r.alpha = cm::make_scalar(1.0); r.beta = cm::make_scalar(0.0);
        r.sparse_feature_order.feature_count = static_cast<cm::u32>(r.k);
        r.sparse_feature_order.feature_axis_identity_version = 1u;
        r.sparse_feature_order.feature_axis_identity = 9u;
        r.dense_feature_order = r.sparse_feature_order;
        const cm::logical_csr_view sp{static_cast<cm::u64>(M), static_cast<cm::u64>(K), static_cast<cm::u64>(nnz), offs.data(),
                                      ucol.data(), decoded.data(), static_cast<cm::u32>(::cellerator::real::value_f32)};
        const cm::logical_dense_view dn{rhs, rhs_rows, static_cast<cm::u64>(N), static_cast<cm::u64>(N),
                                        cm::dense_layout_kind::row_major, static_cast<cm::u32>(::cellerator::real::value_f32)};
        ref->assign(r.m * r.n, 0.0);
        return static_cast<bool>(cm::build_spmm_reference(r, sp, dn, {}, nullptr, ref->data(), ref->size()));
    };
    std::vector<double> ref;
    CHECK(referee(false, w.data(), K, &ref), "referee(forward)");
    {
        const cm::logical_dense_view cand{y.data(), static_cast<cm::u64>(M), static_cast<cm::u64>(N), static_cast<cm::u64>(N),
                                          cm::dense_layout_kind::row_major, static_cast<cm::u32>(::cellerator::real::value_f32)};
        cm::numerical_comparison cmp;
        const bool ok = static_cast<bool>(cm::compare_spmm_reference(ref.data(), ref.size(), cand, {1.0e-4, 1.0e-4, 1.0e-30}, &cmp));
        std::printf("  forward max_abs=%.3e mismatches=%llu\n", cmp.max_absolute_error, static_cast<unsigned long long>(cmp.mismatch_count));
        CHECK(ok && cmp.within_tolerance, "forward result within tolerance of the reference referee");
        cm::determinism_digest d1, d2;
        cm::digest_logical_dense(cand, &d1);
        core::run_prepared_operation(prepared, launch);
        cudaStreamSynchronize(stream);
        std::vector<float> y2(M * N);
        cudaMemcpy(y2.data(), d_y, y2.size() * sizeof(float), cudaMemcpyDeviceToHost);
        const cm::logical_dense_view cand2{y2.data(), static_cast<cm::u64>(M), static_cast<cm::u64>(N), static_cast<cm::u64>(N),
                                           cm::dense_layout_kind::row_major, static_cast<cm::u32>(::cellerator::real::value_f32)};
        cm::digest_logical_dense(cand2, &d2);
        CHECK(cm::same_digest(d1, d2), "deterministic candidate: identical digest on a second run");
    }

    // ---- launch-time rejections by the reference's validate_launch_bindings / by the backend ----
    {
        ex::relation_structure stale = structure;
        stale.epoch = {4u};
        ex::launch_bindings bad = launch;
        bad.structures = &stale;
        CHECK(core::run_prepared_operation(prepared, bad).code == core::operation_status_code::stale_structure,
              "a launch with another structure epoch is stale");
        bad = launch;
        bad.workspace.bytes = 16u;
        const core::operation_status s = core::run_prepared_operation(prepared, bad);
        CHECK(s.code == core::operation_status_code::invalid_launch_bindings &&
                  s.binding == ex::binding_validation_code::insufficient_workspace, "a workspace below the requirement is refused");
        bad = launch;
        bad.stream.device_ordinal = 1;
        CHECK(core::run_prepared_operation(prepared, bad).binding == ex::binding_validation_code::invalid_stream,
              "stream and workspace on different devices are refused");
        ex::value_binding old_value{&plane, {4u}};
        bad = launch;
        bad.values = &old_value;
        CHECK(core::run_prepared_operation(prepared, bad).binding == ex::binding_validation_code::stale_value,
              "a stale value generation is refused");
        ex::biological_operand_view alias_out[1] = {dense_view(d_w, cells, static_cast<std::uint64_t>(M))};
        bad = launch;
        bad.outputs = alias_out;
        CHECK(core::run_prepared_operation(prepared, bad).binding == ex::binding_validation_code::illegal_operand_alias,
              "an output aliasing an input is refused");
    }
    host::release_prepared(&prepared);

    // ---- forward with a composed epilogue: out = gelu_erf(product + bias) -----------------------
    {
        const core::operation_candidate *epi =
            core::find_candidate(registry, host::quantized_csr_forward_epilogue_candidate().identity);
        CHECK(epi != nullptr && (epi->capability_flags & core::candidate_composed_epilogue) != 0u,
              "the composed-epilogue candidate carries its capability flag");
        problem_ids e = make_ids(3u, core::projection_kind::csr, static_cast<std::uint64_t>(nnz));
        host::projection_catalog_entry es = shape;
        es.projection = e.projection.runtime;
        es.epilogue = CB200_EPILOGUE_BIAS_GELU_ERF;
        CHECK(host::register_projection(es), "catalog accepts the epilogue projection");
        core::numeric_policy np = policy_u8(ex::numeric_type::f32);
        np.bias = ex::numeric_type::f32;
        core::prepare_policy no_epilogue;
        no_epilogue.allow_composed_epilogue = false;
        CHECK(core::prepare_candidate(*epi, e.problem, e.structures, e.projection, np, no_epilogue, &prepared).code ==
                  core::operation_status_code::capability_rejected, "a policy without composed epilogues rejects the candidate");
        CHECK(core::prepare_candidate(*fwd, e.problem, e.structures, e.projection, np, {}, &prepared).code ==
                  core::operation_status_code::unsupported_problem, "the plain candidate refuses a projection that composes an epilogue");
        CHECK(core::prepare_candidate(*epi, e.problem, e.structures, e.projection, np, {}, &prepared).code ==
                  core::operation_status_code::unsupported_problem, "a bias epilogue needs the bias as third input");
        e.problem.input_count = 3u;
        st = core::prepare_candidate(*epi, e.problem, e.structures, e.projection, np, {}, &prepared);
        CHECK(static_cast<bool>(st), "prepare_candidate(forward + bias + exact GELU)");
        if (!st) std::printf("  message: %s\n", st.message);

        std::vector<float> bias(N);
        for (auto &v : bias) v = one(rng);
        float *d_bias = to_device(bias);
        ex::relation_structure es_structure = structure;
        es_structure.identity = e.structures.structures[0].runtime;
        ex::value_plane eplane = plane;
        eplane.structure = es_structure.identity;
        ex::value_binding evalue{&eplane, {5u}};
        ex::biological_operand_view in3[3] = {inputs[0], inputs[1], {}};
        in3[0].storage.relation.structure = es_structure.identity;
        in3[0].storage.relation.projection = e.projection.runtime;
        in3[2].kind = ex::operand_kind::dense_tensor;
        in3[2].storage.dense.data = d_bias;
        in3[2].storage.dense.location = dev_loc;
        in3[2].storage.dense.value_type = ex::numeric_type::f32;
        in3[2].storage.dense.rank = 1u;
        in3[2].storage.dense.axes[0] = latent;
        in3[2].storage.dense.shape[0] = static_cast<std::uint64_t>(N);
        in3[2].storage.dense.stride[0] = 1;
        ex::launch_bindings el = launch;
        el.structures = &es_structure;
        el.values = &evalue;
        el.inputs = in3;
        el.input_count = 3u;
        cudaMemset(d_y, 0xff, M * N * sizeof(float));
        st = core::run_prepared_operation(prepared, el);
        CHECK(static_cast<bool>(st), "run_prepared_operation(forward + epilogue)");
        if (!st) std::printf("  message: %s (binding %d)\n", st.message, static_cast<int>(st.binding));
        cudaStreamSynchronize(stream);
        cudaMemcpy(y.data(), d_y, y.size() * sizeof(float), cudaMemcpyDeviceToHost);

        cm::spmm_request r;
        r.m = M; r.k = K; r.n = N; r.sparse_nnz = nnz;
        r.sparse_structure.identity_version = 1u; r.sparse_structure.value = 77u;
        r.dense_rhs_leading_dimension = N; r.output_leading_dimension = N;
        r.sparse_storage_type_code = r.dense_storage_type_code = r.output_storage_type_code = ::cellerator::real::value_f32;
        r.compute_type_code = r.accumulation_type_code = ::cellerator::real::value_f64;
        r.alpha = cm::make_scalar(1.0); r.beta = cm::make_scalar(0.0);
        r.sparse_feature_order.feature_count = static_cast<cm::u32>(K);
        r.sparse_feature_order.feature_axis_identity_version = 1u;
        r.sparse_feature_order.feature_axis_identity = 9u;
        r.dense_feature_order = r.sparse_feature_order;
        r.epilogue.kind = cm::epilogue_kind::bias_gelu_exact_erf;
        r.epilogue.bias_type_code = ::cellerator::real::value_f32;
        r.epilogue.bias_element_count = static_cast<cm::u64>(N);
        const cm::logical_csr_view sp{static_cast<cm::u64>(M), static_cast<cm::u64>(K), static_cast<cm::u64>(nnz), offs.data(),
                                      ucol.data(), decoded.data(), static_cast<cm::u32>(::cellerator::real::value_f32)};
        const cm::logical_dense_view dn{w.data(), static_cast<cm::u64>(K), static_cast<cm::u64>(N), static_cast<cm::u64>(N),
                                        cm::dense_layout_kind::row_major, static_cast<cm::u32>(::cellerator::real::value_f32)};
        std::vector<double> eref(M * N, 0.0);
        CHECK(static_cast<bool>(cm::build_spmm_reference(r, sp, dn, {}, bias.data(), eref.data(), eref.size())),
              "referee(forward + bias + exact GELU)");
        const cm::logical_dense_view cand{y.data(), static_cast<cm::u64>(M), static_cast<cm::u64>(N), static_cast<cm::u64>(N),
                                          cm::dense_layout_kind::row_major, static_cast<cm::u32>(::cellerator::real::value_f32)};
        cm::numerical_comparison cmp;
        const bool ok = static_cast<bool>(cm::compare_spmm_reference(eref.data(), eref.size(), cand, {1.0e-4, 1.0e-4, 1.0e-30}, &cmp));
        std::printf("  forward + epilogue max_abs=%.3e mismatches=%llu\n", cmp.max_absolute_error,
                    static_cast<unsigned long long>(cmp.mismatch_count));
        CHECK(ok && cmp.within_tolerance, "composed epilogue within tolerance of the reference referee");
        el.input_count = 2u;
        CHECK(!static_cast<bool>(core::run_prepared_operation(prepared, el)), "a launch without the bias operand is refused");
        host::release_prepared(&prepared);
        cudaFree(d_bias);
    }

    // ---- forward with the affine output effect: out = alpha * product + beta * out ---------------
    {
        problem_ids a = make_ids(4u, core::projection_kind::csr, static_cast<std::uint64_t>(nnz));
        host::projection_catalog_entry as = shape;
        as.projection = a.projection.runtime;
        as.output_update = ex::output_update_kind::affine_accumulate;
        as.alpha_binding_id = 11u;
        as.beta_binding_id = 12u;
        CHECK(host::register_projection(as), "catalog accepts the affine projection");
        st = core::prepare_candidate(*fwd, a.problem, a.structures, a.projection, policy_u8(ex::numeric_type::f32), {}, &prepared);
        CHECK(static_cast<bool>(st), "prepare_candidate(forward, affine_accumulate)");
        if (!st) std::printf("  message: %s\n", st.message);
        CHECK(prepared.binding_contract.output_effects[0].update == ex::output_update_kind::affine_accumulate &&
                  prepared.binding_contract.output_effects[0].requires_initialized_destination,
              "the contract declares the affine effect and an initialised destination");
        ex::relation_structure a_structure = structure;
        a_structure.identity = a.structures.structures[0].runtime;
        ex::value_plane a_plane = plane;
        a_plane.structure = a_structure.identity;
        ex::value_binding a_value{&a_plane, {5u}};
        ex::biological_operand_view a_in[2] = {inputs[0], inputs[1]};
        a_in[0].storage.relation.structure = a_structure.identity;
        a_in[0].storage.relation.projection = a.projection.runtime;
        std::vector<float> y0(M * N);
        for (auto &v : y0) v = one(rng);
        cudaMemcpy(d_y, y0.data(), y0.size() * sizeof(float), cudaMemcpyHostToDevice);
        ex::launch_bindings al = launch;
        al.structures = &a_structure;
        al.values = &a_value;
        al.inputs = a_in;
        const float alpha = 2.0f;
        const double beta = 0.5; // one scalar of each accepted type
        al.scalars.count = 2u;
        al.scalars.values[0] = {11u, ex::numeric_type::f32, {}, 0u};
        std::memcpy(&al.scalars.values[0].bits, &alpha, sizeof alpha);
        al.scalars.values[1] = {12u, ex::numeric_type::f64, {}, 0u};
        std::memcpy(&al.scalars.values[1].bits, &beta, sizeof beta);
        st = core::run_prepared_operation(prepared, al);
        CHECK(static_cast<bool>(st), "run_prepared_operation(forward, alpha = 2, beta = 0.5)");
        if (!st) std::printf("  message: %s (binding %d)\n", st.message, static_cast<int>(st.binding));
        cudaStreamSynchronize(stream);
        cudaMemcpy(y.data(), d_y, y.size() * sizeof(float), cudaMemcpyDeviceToHost);
        double worst = 0.0; // `ref` still holds the plain product of the forward leg
        for (std::size_t i = 0; i < y.size(); ++i)
            worst = std::max(worst, std::fabs(static_cast<double>(y[i]) - (2.0 * ref[i] + 0.5 * static_cast<double>(y0[i]))));
        std::printf("  affine forward max_abs=%.3e\n", worst);
        CHECK(worst <= 1.0e-4, "alpha * product + beta * out within tolerance of the referee's product");
        ex::launch_bindings missing = al;
        missing.scalars.count = 1u;
        CHECK(!static_cast<bool>(core::run_prepared_operation(prepared, missing)), "a launch without the beta scalar is refused");
        host::release_prepared(&prepared);
    }

    // ---- transpose candidate -------------------------------------------------------------------
    {
        problem_ids t = make_ids(1u, core::projection_kind::transpose_or_backward, static_cast<std::uint64_t>(nnz));
        host::projection_catalog_entry ts = shape;
        ts.projection = t.projection.runtime;
        ts.projection_kind = CB200_PROJECTION_TRANSPOSE;
        host::register_projection(ts);
        core::prepared_operation pt{};
        st = core::prepare_candidate(*tr, t.problem, t.structures, t.projection, policy_u8(ex::numeric_type::f32), {}, &pt);
        CHECK(static_cast<bool>(st), "prepare_candidate(transpose)");
        ex::relation_structure s2{t.structures.structures[0].runtime, {3u}, cells, genes, {1u, 1u}, static_cast<std::uint64_t>(nnz)};
        ex::value_plane plane2 = plane;
        plane2.structure = s2.identity;
        ex::value_binding v2{&plane2, {5u}};
        ex::biological_operand_view in2[2] = {inputs[0], dense_view(d_g, cells, static_cast<std::uint64_t>(M))};
        in2[0].storage.relation.structure = s2.identity;
        in2[0].storage.relation.projection = t.projection.runtime;
        ex::biological_operand_view out2[1] = {dense_view(d_gt, genes, static_cast<std::uint64_t>(K))};
        ex::launch_bindings l2 = launch;
        l2.structures = &s2; l2.inputs = in2; l2.outputs = out2; l2.values = &v2;
        st = core::run_prepared_operation(pt, l2);
        CHECK(static_cast<bool>(st), "run_prepared_operation(transpose)");
        if (!st) std::printf("  message: %s (binding %d)\n", st.message, static_cast<int>(st.binding));
        cudaStreamSynchronize(stream);
        std::vector<float> gt(K * N);
        cudaMemcpy(gt.data(), d_gt, gt.size() * sizeof(float), cudaMemcpyDeviceToHost);
        CHECK(referee(true, g.data(), M, &ref), "referee(transpose)");
        const cm::logical_dense_view cand{gt.data(), static_cast<cm::u64>(K), static_cast<cm::u64>(N), static_cast<cm::u64>(N),
                                          cm::dense_layout_kind::row_major, static_cast<cm::u32>(::cellerator::real::value_f32)};
        cm::numerical_comparison cmp;
        const bool ok = static_cast<bool>(cm::compare_spmm_reference(ref.data(), ref.size(), cand, {1.0e-3, 1.0e-4, 1.0e-30}, &cmp));
        std::printf("  transpose max_abs=%.3e mismatches=%llu\n", cmp.max_absolute_error, static_cast<unsigned long long>(cmp.mismatch_count));
        CHECK(ok && cmp.within_tolerance, "transpose result within tolerance of the reference referee");
        host::release_prepared(&pt);
    }

    // ---- transpose with the matrix handed to prepare: tensor-core schedule, split products --------
    {
        problem_ids t = make_ids(2u, core::projection_kind::transpose_or_backward, static_cast<std::uint64_t>(nnz));
        cb200_qcsr dm{};
        dm.version = CB200_ABI_VERSION; dm.size = sizeof dm; dm.rows = M; dm.cols = K; dm.nnz = nnz; dm.bits = 8;
        dm.policy = CB200_DECODE_PER_GENE_AFFINE; dm.row_ptr = d_row_ptr; dm.col_idx = d_col; dm.packed_values = d_codes;
        dm.scales = d_scales; dm.offsets = d_offsets;
        host::projection_catalog_entry ts = shape;
        ts.projection = t.projection.runtime;
        ts.projection_kind = CB200_PROJECTION_TRANSPOSE;
        ts.device_matrix = &dm;
        ts.device_matrix_generation = {5u}; // the generation of `plane`
        ts.schedule_hint = "tensor_blocked"; // the matrix is far below the size prepare would pick it for
        // the copy lives in memory the execution session reserved before sealing (prepared state borrows it,
        // OPERATION_CORE.md:17-25): sized by the backend, handed over through the catalog entry
        cb200_spmm_problem sizing{};
        sizing.version = CB200_ABI_VERSION; sizing.size = sizeof sizing; sizing.projection = CB200_PROJECTION_TRANSPOSE;
        sizing.m = M; sizing.k = K; sizing.n = N; sizing.nnz = nnz; sizing.bits = 8; sizing.policy = CB200_DECODE_PER_GENE_AFFINE;
        sizing.dense_dtype = CB200_DTYPE_F32; sizing.structure_epoch = 3u; sizing.multiply = CB200_DTYPE_F32; sizing.device_matrix = &dm;
        sizing.schedule_hint = "tensor_blocked";
        std::uint64_t persistent_need = 0u;
        CHECK(cb200_spmm_persistent_requirement(&sizing, &persistent_need) == CB200_STATUS_SUCCESS && persistent_need >= static_cast<std::uint64_t>(nnz) * 8u,
              "the backend sizes the persistent memory of the split-product transpose (two words per entry)");
        cb200_session_options sopt{};
        sopt.version = CB200_ABI_VERSION; sopt.size = sizeof sopt; sopt.device = 0; sopt.owned_stream_count = 1u;
        cb200_session *session = nullptr;
        void *session_block = nullptr;
        CHECK(cb200_session_create(&sopt, &session) == CB200_STATUS_SUCCESS &&
                  cb200_session_reserve_persistent_as(session, CB200_LIFETIME_STRUCTURE, persistent_need, &session_block) == CB200_STATUS_SUCCESS &&
                  cb200_session_seal(session) == CB200_STATUS_SUCCESS,
              "session: reserve the persistent block, then seal");
        const cb200_launch_binding bound = cb200_session_bind(session, 0u, 0u);
        ts.persistent = session_block;
        ts.persistent_bytes = persistent_need;
        ts.prepare_stream = bound.stream;
        std::size_t free_before = 0, free_after = 0, total_mem = 0;
        cudaMemGetInfo(&free_before, &total_mem);
        host::register_projection(ts);
        core::prepared_operation pt{};
        core::prepare_policy with_preprocessing;
        with_preprocessing.allow_persistent_preprocessing = true;
        st = core::prepare_candidate(*tr, t.problem, t.structures, t.projection, policy_u8(ex::numeric_type::f32),
                                     with_preprocessing, &pt);
        CHECK(static_cast<bool>(st), "prepare_candidate(transpose, matrix handed to prepare)");
        if (!st) std::printf("  message: %s\n", st.message);
        CHECK(std::strcmp(host::prepared_schedule(pt), "tensor_blocked_x3") == 0, "fp32 products + matrix at prepare -> split-product tensor schedule");
        cudaMemGetInfo(&free_after, &total_mem);
        CHECK(free_after == free_before, "prepare built its copy inside the session's block: no device memory was allocated");
        CHECK(pt.binding_contract.workspace.minimum_bytes > 4096u, "the schedule reports its workspace (bf16 records of G)");
        void *d_ws2 = nullptr;
        const std::size_t ws2 = static_cast<std::size_t>(pt.binding_contract.workspace.minimum_bytes);
        cudaMalloc(&d_ws2, ws2);
        ex::relation_structure s2{t.structures.structures[0].runtime, {3u}, cells, genes, {1u, 1u}, static_cast<std::uint64_t>(nnz)};
        ex::value_plane plane2 = plane;
        plane2.structure = s2.identity;
        ex::value_binding v2{&plane2, {5u}};
        ex::biological_operand_view in2[2] = {inputs[0], dense_view(d_g, cells, static_cast<std::uint64_t>(M))};
        in2[0].storage.relation.structure = s2.identity;
        in2[0].storage.relation.projection = t.projection.runtime;
        ex::biological_operand_view out2[1] = {dense_view(d_gt, genes, static_cast<std::uint64_t>(K))};
        ex::launch_bindings l2 = launch;
        l2.structures = &s2; l2.inputs = in2; l2.outputs = out2; l2.values = &v2;
        l2.workspace = {d_ws2, ws2, dev_loc};
        st = core::run_prepared_operation(pt, l2);
        CHECK(static_cast<bool>(st), "run_prepared_operation(transpose, split products)");
        if (!st) std::printf("  message: %s (binding %d)\n", st.message, static_cast<int>(st.binding));
        cudaStreamSynchronize(stream);
        std::vector<float> gt(K * N);
        cudaMemcpy(gt.data(), d_gt, gt.size() * sizeof(float), cudaMemcpyDeviceToHost);
        CHECK(referee(true, g.data(), M, &ref), "referee(transpose)");
        // the contract's bound for an fp32 dense operand: 1e-4 * ||gene column||_1 * max|G|
        std::vector<double> col_l1(K, 0.0);
        for (std::int64_t i = 0; i < nnz; ++i) col_l1[col[i]] += std::fabs(static_cast<double>(decoded[i]));
        double gmax = 0.0, worst = 0.0;
        for (float v : g) gmax = std::max(gmax, static_cast<double>(std::fabs(v)));
        for (std::int64_t gene = 0; gene < K; ++gene)
            for (std::int64_t c = 0; c < N; ++c) {
                const double scale = col_l1[gene] * gmax + 1e-30;
                worst = std::max(worst, std::fabs(static_cast<double>(gt[gene * N + c]) - ref[gene * N + c]) / scale);
            }
        std::printf("  transpose (split products) max |d| / (||column||_1 max|G|) = %.3e\n", worst);
        CHECK(worst <= 1.0e-4, "split-product transpose within the fp32 bound of the reference referee's result");
        // new values under the same structure: the copy prepare built is of generation 5
        plane2.generation = {6u};
        ex::value_binding v3{&plane2, {6u}};
        l2.values = &v3;
        const core::operation_status newer = core::run_prepared_operation(pt, l2);
        CHECK(newer.code == core::operation_status_code::invalid_launch_bindings &&
                  newer.binding == ex::binding_validation_code::stale_value,
              "a launch with a newer value generation is refused by an operation that keeps a copy of the values");
        // ---- the ordered transpose: a deterministic policy selects it, two runs agree in every bit ----
        {
            const core::operation_candidate *ord =
                core::find_candidate(registry, host::quantized_csr_transpose_ordered_candidate().identity);
            CHECK(ord != nullptr && (ord->capability_flags & core::candidate_deterministic) != 0u &&
                      (ord->capability_flags & core::candidate_persistent_preprocessing) != 0u,
                  "the ordered transpose claims determinism and persistent preprocessing");
            core::prepare_policy det_only;
            det_only.deterministic = true;
            det_only.allow_persistent_preprocessing = false;
            core::prepared_operation po{};
            CHECK(core::prepare_candidate(*ord, t.problem, t.structures, t.projection, policy_u8(ex::numeric_type::f32), det_only, &po).code ==
                      core::operation_status_code::capability_rejected,
                  "without persistent preprocessing the ordered transpose is rejected");
            core::prepare_policy det_pre = with_preprocessing;
            det_pre.deterministic = true;
            ts.persistent = nullptr; // the session's block holds the split-product copy: this operation allocates its own
            ts.persistent_bytes = 0u;
            ts.schedule_hint = nullptr;
            host::register_projection(ts);
            st = core::prepare_candidate(*ord, t.problem, t.structures, t.projection, policy_u8(ex::numeric_type::f32), det_pre, &po);
            CHECK(static_cast<bool>(st), "prepare_candidate(ordered transpose, deterministic policy)");
            if (!st) std::printf("  message: %s\n", st.message);
            CHECK(std::strcmp(host::prepared_schedule(po), "gene_gather") == 0, "deterministic transpose -> gather schedule");
            plane2.generation = {5u};
            l2.values = &v2;
            std::vector<float> first(K * N), second(K * N);
            st = core::run_prepared_operation(po, l2);
            CHECK(static_cast<bool>(st), "run_prepared_operation(ordered transpose)");
            if (!st) std::printf("  message: %s (binding %d)\n", st.message, static_cast<int>(st.binding));
            cudaStreamSynchronize(stream);
            cudaMemcpy(first.data(), d_gt, first.size() * sizeof(float), cudaMemcpyDeviceToHost);
            cudaMemset(d_gt, 0xff, first.size() * sizeof(float));
            st = core::run_prepared_operation(po, l2);
            cudaStreamSynchronize(stream);
            cudaMemcpy(second.data(), d_gt, second.size() * sizeof(float), cudaMemcpyDeviceToHost);
            CHECK(static_cast<bool>(st) && std::memcmp(first.data(), second.data(), first.size() * sizeof(float)) == 0,
                  "ordered transpose: the second run repeats every bit of the first");
            double worst_ordered = 0.0;
            for (std::int64_t gene = 0; gene < K; ++gene)
                for (std::int64_t c = 0; c < N; ++c)
                    worst_ordered = std::max(worst_ordered, std::fabs(static_cast<double>(first[gene * N + c]) - ref[gene * N + c]) /
                                                                (col_l1[gene] * gmax + 1e-30));
            std::printf("  transpose (ordered) max |d| / (||column||_1 max|G|) = %.3e\n", worst_ordered);
            CHECK(worst_ordered <= 1.0e-4, "ordered transpose within the fp32 bound of the reference referee's result");
            host::release_prepared(&po);
            // the same candidate with the tensor_blocked variant: the tensor-core transpose, whose CTAs' sums are added in a
            // fixed order, under the same deterministic policy
            core::projection_key tensor_variant = t.projection;
            tensor_variant.variant = host::schedule_tensor_blocked;
            core::prepared_operation pb{};
            st = core::prepare_candidate(*ord, t.problem, t.structures, tensor_variant, policy_u8(ex::numeric_type::f32), det_pre, &pb);
            CHECK(static_cast<bool>(st), "prepare_candidate(ordered transpose, tensor_blocked variant, deterministic policy)");
            if (!st) std::printf("  message: %s\n", st.message);
            CHECK(std::strcmp(host::prepared_schedule(pb), "tensor_blocked_x3") == 0, "deterministic transpose, tensor_blocked variant -> split-product tensor schedule");
            ex::launch_bindings l3 = l2;
            l3.structures = l2.structures;
            cudaMemset(d_gt, 0xff, first.size() * sizeof(float));
            st = core::run_prepared_operation(pb, l3);
            CHECK(static_cast<bool>(st), "run_prepared_operation(ordered transpose, tensor_blocked variant)");
            if (!st) std::printf("  message: %s (binding %d)\n", st.message, static_cast<int>(st.binding));
            cudaStreamSynchronize(stream);
            cudaMemcpy(first.data(), d_gt, first.size() * sizeof(float), cudaMemcpyDeviceToHost);
            cudaMemset(d_gt, 0xff, first.size() * sizeof(float));
            st = core::run_prepared_operation(pb, l3);
            cudaStreamSynchronize(stream);
            cudaMemcpy(second.data(), d_gt, second.size() * sizeof(float), cudaMemcpyDeviceToHost);
            CHECK(static_cast<bool>(st) && std::memcmp(first.data(), second.data(), first.size() * sizeof(float)) == 0,
                  "tensor transpose under the deterministic policy: the second run repeats every bit of the first");
            double worst_tensor = 0.0;
            for (std::int64_t gene = 0; gene < K; ++gene)
                for (std::int64_t c = 0; c < N; ++c)
                    worst_tensor = std::max(worst_tensor, std::fabs(static_cast<double>(first[gene * N + c]) - ref[gene * N + c]) /
                                                              (col_l1[gene] * gmax + 1e-30));
            std::printf("  transpose (ordered candidate, tensor_blocked variant) max |d| / (||column||_1 max|G|) = %.3e\n", worst_tensor);
            CHECK(worst_tensor <= 1.0e-4, "tensor transpose under the deterministic policy within the fp32 bound");
            host::release_prepared(&pb);
        }
        host::release_prepared(&pt);
        cudaFree(d_ws2);
        cb200_session_destroy(session); // the owner of the block outlived the prepared operations built in it
    }

    std::printf("%s: %d failure(s)\n", g_failures ? "FAILED" : "OK", g_failures);
    return g_failures ? 1 : 0;
}
