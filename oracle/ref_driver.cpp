// Test infrastructure, not product code.
//
// C entry points over the UNMODIFIED reference (BL-GS/Spy) CPU path. This file
// is compiled together with the reference's own sources (taken from the
// reference checkout at build time, never copied) into oracle/_ref/libspy_ref.so.
// It is used to (1) pin the plain-C restatement in spy_oracle.c, (2) generate
// the golden fixtures under tests/golden/, and (3) time the reference's CPU
// backend as the baseline next to the GPU numbers.
//
// The generate loop mirrors AutoModelGenerator::generate
// (app/cli/include/cli.h:60-129) but takes raw token ids instead of a prompt
// string; the backend/loader/distributor wiring mirrors main
// (app/cli/src/cli.cpp:12-49) with the CLI's default hyper-parameters
// (app/cli/include/cmdline.h:125-141).

#include <chrono>
#include <condition_variable>
#include <cstdint>
#include <cstring>
#include <map>
#include <memory>
#include <mutex>
#include <string>
#include <vector>

#include "util/log/logger.h"
#include "backend/backend.h"
#include "default_backend.h"
#include "loader/loader.h"
#include "llm/model/model.h"
#include "llm/sampler/sampler.h"
#include "distributor/distributor.h"
#include "operator/operator.h"
#include "graph/graph.h"
#include "number/lookup_table.h"
#include "simd/vec_convert.h"
#include "simd/vec_dot.h"

using namespace spy;

namespace {

std::mutex g_mutex;
std::map<int, std::unique_ptr<Backend>> g_backends;
bool g_logger_ready = false;

#ifdef SPY_BACKEND_CUDA
/// the sm_100a backend behind the reference's own factory hook ("gpu:b200"); a fresh instance per call, so that
/// the constants of one model file never outlive its mapping
std::unique_ptr<Backend> g_device_backend;
/// plan_model: path of the GGUF file for the adapter's plan mode (steps served from the fused step plan), or null for
/// operator-by-operator submission
Backend *device_backend(const char *plan_model, int num_context) {
	std::lock_guard<std::mutex> guard(g_mutex);
	if (!g_logger_ready) {
		LogParam log_param;
		log_param.log_level = "error";
		init_logger_format(log_param);
		g_logger_ready = true;
	}
	BackendFactory factory;
	ConfigTable config;
	if (plan_model != nullptr) { config.add("model", plan_model); config.add("num_context", std::to_string(num_context)); }
	g_device_backend.reset();
	g_device_backend = factory.init_backend("gpu:b200", config);
	return g_device_backend.get();
}
#endif

Backend *backend_for(int num_thread) {
	std::lock_guard<std::mutex> guard(g_mutex);
	if (!g_logger_ready) {
		LogParam log_param;
		log_param.log_level = "error";
		init_logger_format(log_param);
		g_logger_ready = true;
	}
	auto iter = g_backends.find(num_thread);
	if (iter != g_backends.end()) { return iter->second.get(); }
	BackendFactory factory;
	ConfigTable config;
	config.add("num_thread", std::to_string(num_thread));
	auto backend = factory.init_backend("cpu:default", config);
	Backend *raw = backend.get();
	g_backends.emplace(num_thread, std::move(backend));
	return raw;
}

HyperParam default_hyper_param(uint32_t num_context) {
	return HyperParam {
		.num_context       = num_context,
		.rope_type         = RopeType::None,
		.rope_scaling_type = HyperParam::parse_rope_scaling_type("unspecified"),
		.rope_pooling_type = HyperParam::parse_pooling_type("unspecified"),
		.rope_freq_base    = 0.0F,
		.rope_freq_scale   = 0.0F,
		.yarn_ext_factor   = -1.0F,
		.yarn_attn_factor  = 1.0F,
		.yarn_beta_fast    = 32.0F,
		.yarn_beta_slow    = 1.0F,
		.yarn_orig_ctx     = 0,
	};
}

struct Waiter {
	std::mutex              m;
	std::condition_variable cv;
	bool                    done = false;

	void signal() { { std::lock_guard<std::mutex> g(m); done = true; } cv.notify_all(); }
	void wait()   { std::unique_lock<std::mutex> g(m); cv.wait(g, [this] { return done; }); }
};

}  // namespace

extern "C" {

/// Tensor descriptor passed across the C boundary: number_type follows the
/// reference's NumberType numbering; nb[] are byte strides (all zero = contiguous).
struct spy_ref_tensor {
	int32_t number_type;
	int32_t dim;
	int64_t ne[4];
	int64_t nb[4];
	void *  data;
};

struct spy_ref_op_param {
	float   scale;        // Softmax
	float   eps;          // NormRMS
	int32_t rope_mode;    // Rope
	int32_t num_past;
	int32_t num_dim;
	int32_t num_context;
	int32_t num_origin_context;
	float   freq_base;
	float   freq_scale;
	float   extend_factor;
	float   attention_factor;
	float   beta_fast;
	float   beta_slow;
};

int spy_ref_init(int num_thread) { return backend_for(num_thread) != nullptr ? 0 : 1; }

/// Quantizator<FP32,Q8_0>::transform (backend/host/include/simd/vec_convert.h:178-261).
void spy_ref_quantize_q8_0(const float *x, int64_t n, void *out) {
	cpu::Quantizator<NumberType::FP32, NumberType::Q8_0>::transform(x, static_cast<block_q8_0_t *>(out), n);
}

/// Quantizator<FP32,FP16>::transform (vec_convert.h:39-65).
void spy_ref_quantize_f16(const float *x, int64_t n, uint16_t *out) {
	cpu::Quantizator<NumberType::FP32, NumberType::FP16>::transform(x, out, n);
}

/// Dot<...>::exec (backend/host/include/simd/vec_dot.h:42-205). kind: 0 = Q4_0xQ8_0, 1 = Q8_0xQ8_0, 2 = F16xF16.
float spy_ref_dot(int kind, const void *w, const void *x, int64_t n) {
	switch (kind) {
	case 0: return cpu::Dot<NumberType::Q4_0, NumberType::Q8_0>::exec_raw(w, x, n);
	case 1: return cpu::Dot<NumberType::Q8_0, NumberType::Q8_0>::exec_raw(w, x, n);
	case 2: return cpu::Dot<NumberType::FP16, NumberType::FP16>::exec_raw(w, x, n);
	default: return 0.0F;
	}
}

/// The reference's 65 536-entry fp16 tables (orchestration/include/number/lookup_table.h:12-54).
void spy_ref_tables(float *fp32_table, float *silu_table, float *exp_table) {
	for (uint32_t k = 0; k < 65536; ++k) {
		const uint16_t key = static_cast<uint16_t>(k);
		if (fp32_table != nullptr) { fp32_table[k] = LOOK_UP_TABLE.fp32(key); }
		if (silu_table != nullptr) { silu_table[k] = LOOK_UP_TABLE.silu(key); }
		if (exp_table  != nullptr) { exp_table[k]  = LOOK_UP_TABLE.exp(key); }
	}
}

static Shape make_shape(const spy_ref_tensor &t) {
	const NumberType type = static_cast<NumberType>(t.number_type);
	const Shape::DimensionArray ne{ t.ne[0], t.ne[1], t.ne[2], t.ne[3] };
	const bool contiguous = (t.nb[0] == 0 && t.nb[1] == 0 && t.nb[2] == 0 && t.nb[3] == 0);
	if (contiguous) { return Shape(static_cast<uint32_t>(t.dim), ne, type); }
	const Shape::DimensionArray nb{ t.nb[0], t.nb[1], t.nb[2], t.nb[3] };
	return Shape(static_cast<uint32_t>(t.dim), ne, nb, type);
}

/// Runs one operator of the reference CPU backend (DefaultCPUBackend::submit,
/// backend/host/include/default_backend.h:164-182) on caller-owned buffers.
/// `out->data` must be large enough; `out->ne/nb/number_type` are filled from
/// the operator's own shape inference. For Copy the destination is in[1].
int spy_ref_run_op(int op_type, int num_in, const spy_ref_tensor *in, spy_ref_tensor *out,
		const spy_ref_op_param *param, int num_thread) {
	Backend *backend = backend_for(num_thread);

	GraphStorage storage;
	Graph graph(0, storage);

	const DataNodeProperty in_prop { .node_type = DataNodeType::IO, .layer_id = -1, .expert_id = -1 };
	const DataNodeProperty out_prop{ .node_type = DataNodeType::IO, .layer_id = -1, .expert_id = -1 };

	std::vector<DataNode *> inputs;
	for (int i = 0; i < num_in; ++i) {
		DataNode &node = graph.alloc_node<DataNode>(in_prop, make_shape(in[i]), in[i].data);
		node.name = "in" + std::to_string(i);
		inputs.push_back(std::addressof(node));
	}

	OperatorNode *op_node = nullptr;
	DataNode *result = nullptr;
	const OperatorType type = static_cast<OperatorType>(op_type);

	auto unary = [&]<OperatorType T>() {
		auto &op = graph.alloc_node<OperatorDefinition<T>>();
		result   = op.set_name("op").set_input(inputs[0]).deduce(graph, out_prop);
		op_node  = std::addressof(op);
	};
	auto binary = [&]<OperatorType T>() {
		auto &op = graph.alloc_node<OperatorDefinition<T>>();
		result   = op.set_name("op").set_input(inputs[0], inputs[1]).deduce(graph, out_prop);
		op_node  = std::addressof(op);
	};

	switch (type) {
	case OperatorType::MatMul: binary.template operator()<OperatorType::MatMul>(); break;
	case OperatorType::Add:    binary.template operator()<OperatorType::Add>();    break;
	case OperatorType::Mul:    binary.template operator()<OperatorType::Mul>();    break;
	case OperatorType::GetRow: binary.template operator()<OperatorType::GetRow>(); break;
	case OperatorType::Copy:   binary.template operator()<OperatorType::Copy>();   break;
	case OperatorType::Silu:   unary.template operator()<OperatorType::Silu>();    break;
	case OperatorType::Contiguous: unary.template operator()<OperatorType::Contiguous>(); break;
	case OperatorType::Softmax: {
		auto &op = graph.alloc_node<OperatorDefinition<OperatorType::Softmax>>(SoftmaxParam{ .scale = param->scale });
		result   = op.set_name("op").set_input(inputs[0], inputs[1]).deduce(graph, out_prop);
		op_node  = std::addressof(op);
	} break;
	case OperatorType::NormRMS: {
		auto &op = graph.alloc_node<OperatorDefinition<OperatorType::NormRMS>>(NormRMSParam{ .eps = param->eps });
		result   = op.set_name("op").set_input(inputs[0]).deduce(graph, out_prop);
		op_node  = std::addressof(op);
	} break;
	case OperatorType::Rope: {
		const RopeParam rope {
			.mode = static_cast<RopeType>(param->rope_mode),
			.num_past = param->num_past, .num_dim = param->num_dim,
			.num_context = param->num_context, .num_origin_context = param->num_origin_context,
			.freq_base = param->freq_base, .freq_scale = param->freq_scale,
			.extend_factor = param->extend_factor, .attention_factor = param->attention_factor,
			.beta_fast = param->beta_fast, .beta_slow = param->beta_slow,
			.xpos_base = 0.0F, .xpos_down = false,
		};
		auto &op = graph.alloc_node<OperatorDefinition<OperatorType::Rope>>(rope);
		result   = op.set_name("op").set_input(inputs[0], inputs[1]).deduce(graph, out_prop);
		op_node  = std::addressof(op);
	} break;
	default:
		return 2;
	}

	op_node->propagate();
	result->tensor.set_data_ptr(out->data);

	Waiter waiter;
	backend->submit(op_node, [&waiter] { waiter.signal(); });
	waiter.wait();

	const Shape &shape = result->tensor.get_shape();
	out->number_type = static_cast<int32_t>(shape.number_type);
	out->dim = static_cast<int32_t>(shape.dim);
	for (int i = 0; i < 4; ++i) { out->ne[i] = shape.elements[i]; out->nb[i] = shape.bytes[i]; }
	return 0;
}

/// Prefill + greedy decode through the reference's own model graph, scheduler
/// and CPU backend. step 0 executes all prompt tokens, later steps one token.
///   out_ids    [n_predict]            greedy token per step
///   out_logits [n_predict * n_vocab]  last-token logits per step (may be null)
///   step_ms    [n_predict]            wall time of distributor->execute() per step (may be null)
/// Returns the vocabulary size, or a negative value on failure.
/// num_thread < 0 selects the device backend (only in the build with -DSPY_BACKEND_CUDA, which links the adapter
/// spy_b200/adapter/b200_backend.cpp and libspyb200.so): the reference's graph builder, scheduler, loader and sampler
/// then run unchanged on top of spy::gpu::B200Backend.
int spy_ref_generate(const char *gguf_path, const int32_t *prompt, int n_prompt, int n_predict, int num_context,
		int num_thread, int warmup, int32_t *out_ids, float *out_logits, double *step_ms) {
#ifdef SPY_BACKEND_CUDA
	// num_thread -1: operator by operator; num_thread -2: the adapter's plan mode
	Backend *backend = (num_thread < 0) ? device_backend(num_thread == -2 ? gguf_path : nullptr, num_context) : backend_for(num_thread);
#else
	if (num_thread < 0) { return -2; }
	Backend *backend = backend_for(num_thread);
#endif

	std::unique_ptr<ModelLoader> loader = ModelLoaderFactory::build_model_loader("simple", gguf_path);
	std::unique_ptr<Model> model = ModelBuilder::build_model(loader->context, default_hyper_param(num_context));
	std::unique_ptr<Sampler> sampler = SamplerFactory::build_sampler(SamplerType::Greedy);
	std::unique_ptr<GraphDistributor> distributor = GraphDistributorFactory::build_graph_distributor("simple", loader.get());
	loader->preload();

	GraphStorage storage;
	Graph graph(0, storage);
	distributor->add_backend(backend, "greedy");

	const size_t num_vocab = model->get_info().num_vocab;

	ModelIO model_io;
	for (int i = 0; i < n_prompt; ++i) { model_io.add(prompt[i], i, { 0 }, false); }
	model_io.enable_logits.back() = true;

	model->build_graph(loader->context, graph, model_io);
	distributor->prepare_graph(std::addressof(graph));

	if (warmup != 0) { distributor->execute(); }

	int32_t cur_pos = 0;
	for (int step = 0; step < n_predict; ++step) {
		const size_t num_token = model_io.num_token();

		const auto t0 = std::chrono::steady_clock::now();
		distributor->execute();
		const auto t1 = std::chrono::steady_clock::now();
		if (step_ms != nullptr) { step_ms[step] = std::chrono::duration<double, std::milli>(t1 - t0).count(); }

		const float *logits = model_io.logits.data() + model_io.logits.size() - num_vocab;
		if (out_logits != nullptr) { std::memcpy(out_logits + static_cast<size_t>(step) * num_vocab, logits, num_vocab * sizeof(float)); }

		TokenCandidateArray candidates(num_vocab);
		for (size_t id = 0; id < num_vocab; ++id) {
			candidates[id] = { .token_id = static_cast<TokenID>(id), .logit = logits[id] };
		}
		const TokenID next = sampler->sample(candidates);
		out_ids[step] = next;

		model_io.reset();
		cur_pos += static_cast<int32_t>(num_token);
		model_io.add(next, cur_pos, { 0 }, true);
		model->propagate(graph, model_io);
	}
	return static_cast<int>(num_vocab);
}

}  // extern "C"
