#include "b200_backend.h"

namespace spy::gpu {

	static spyb_tensor to_pod(const DataNode *node, void *data_override = nullptr) {
		const Tensor &tensor = node->tensor;
		const Shape  &shape  = tensor.get_shape();
		spyb_tensor pod{};
		pod.number_type = static_cast<int32_t>(shape.number_type);
		pod.dim         = shape.dim;
		for (int i = 0; i < 4; ++i) { pod.elements[i] = shape.elements[i]; pod.bytes[i] = shape.bytes[i]; }
		pod.data      = (data_override != nullptr) ? data_override : tensor.get();
		pod.node_type = static_cast<int32_t>(node->node_prop.node_type);
		return pod;
	}

	B200Backend::B200Backend(const BackendFactory::BackendConfiguration &config): Backend(BackendType::Device) {
		spyb_config pod{};
		pod.device_id   = device_id_ = config.parse_or("device_id", 0);
		pod.tp_size     = config.parse_or("tp_size", 1);
		pod.tp_rank     = config.parse_or("tp_rank", 0);
		pod.use_pdl     = config.parse_or("use_pdl", 1);
		pod.use_graph   = config.parse_or("graph_replay", 1);
		pod.arena_bytes = config.parse_or<uint64_t>("arena_bytes", 0);
		const spyb_status status = spyb_create(&pod, &handle_);
		spy_assert(status == SPYB_SUCCESS && handle_ != nullptr, "Failed to create the B200 backend on device {}: no CPU fallback exists", device_id_);
		plan_path_    = config.get_or("model", "");
		plan_context_ = config.parse_or("num_context", 512);
		plan_enabled_ = !plan_path_.empty() && config.parse_or("plan", 1) != 0;
	}

	B200Backend::~B200Backend() noexcept {
		if (plan_model_ != nullptr) { spyb_model_free(plan_model_); }
		spyb_destroy(handle_);
	}

	/*!
	 * @brief Plan mode: serve the node from the fused step plan. Returns false when the node has to take the
	 * operator-by-operator path (plan mode off, or the model is one the step plan does not cover).
	 * @note The step's graph is the one LLAMAModel::build_graph emits (model/src/llm/model/llama.cpp:123-222): the token
	 * ids enter through GetRow on the embedding table (plugin/inout.cpp:5-30), the position through the Rope parameters
	 * (plugin/attention.cpp:64-97), and the only node whose output lives in host memory is the logits MatMul
	 * (plugin/inout.cpp:61-75). Its output tensor holds one column of logits per token of the step; like the reference's
	 * generate loop (app/cli/include/cli.h:103-105) only the last column is filled.
	 */
	bool B200Backend::submit_planned(OperatorNode *op_node_ptr) {
		if (!plan_enabled_) { return false; }
		if (!plan_tried_) {
			plan_tried_ = true;
			if (spyb_model_load_gguf(handle_, plan_path_.c_str(), plan_context_, &plan_model_) != SPYB_SUCCESS) { plan_model_ = nullptr; }
		}
		if (plan_model_ == nullptr) { return false; }

		DataNode *output_node = (op_node_ptr->num_output() > 0) ? op_node_ptr->output_data(0) : nullptr;
		const OperatorType op_type = op_node_ptr->op_type;
		if (op_type == OperatorType::GetRow && op_node_ptr->num_input() >= 2 && op_node_ptr->input_data(1)->node_prop.node_type == DataNodeType::IO) {
			const Tensor &ids = op_node_ptr->input_data(1)->tensor;
			plan_ids_       = static_cast<const int32_t *>(ids.get());
			plan_num_token_ = static_cast<int>(ids.get_shape().total_element());
			plan_num_past_  = -1;
		} else if (op_type == OperatorType::Rope && plan_num_past_ < 0) {
			plan_num_past_ = static_cast<OperatorDefinition<OperatorType::Rope> *>(op_node_ptr)->params.get_val().num_past;
		} else if (output_node != nullptr && is_view(op_type)) {
			// the scheduler leaves the output pointer of view-type operators to the backend (backend/host/operator/view.cpp:224-276)
			if (op_type == OperatorType::Copy) { output_node->tensor.set_data_ptr(op_node_ptr->input_data(1)->tensor.get()); }
			else {
				uint8_t *base = static_cast<uint8_t *>(op_node_ptr->input_data(0)->tensor.get());
				const int64_t offset = (op_type == OperatorType::View) ? static_cast<OperatorDefinition<OperatorType::View> *>(op_node_ptr)->params.get_val().offset : 0;
				output_node->tensor.set_data_ptr(base + offset);
			}
		}
		if (output_node != nullptr && output_node->node_prop.node_type == DataNodeType::IO) {   // the logits: run the step
			spy_assert(plan_ids_ != nullptr && plan_num_token_ > 0 && plan_num_past_ >= 0, "B200 backend: the step plan saw no token ids / position before the logits node");
			spyb_model_info info{};
			spyb_model_info_get(plan_model_, &info);
			float *logits = static_cast<float *>(output_node->tensor.get()) + static_cast<size_t>(plan_num_token_ - 1) * info.n_vocab;
			const spyb_status status = spyb_model_eval(plan_model_, plan_ids_, plan_num_token_, plan_num_past_, logits);
			spy_assert(status == SPYB_SUCCESS, "B200 backend (step plan): {}", spyb_last_error(handle_));
			plan_ids_ = nullptr; plan_num_token_ = 0; plan_num_past_ = -1;
		}
		return true;
	}

	void *B200Backend::alloc_memory(size_t size) {
		void *ptr = spyb_alloc(handle_, size);
		spy_assert(ptr != nullptr, "B200 backend: {}", spyb_last_error(handle_));
		return ptr;
	}

	/*!
	 * @brief Translate the node into the plain-C descriptor and enqueue it on the backend's stream.
	 * @note Constant operands arrive as host spans of the loader's mmap
	 * (backend/distributor/include/scheduler/default_scheduler.h:141-165); they are uploaded once, by name,
	 * and replaced by their device copy. Every operator is stream-ordered, so the callback (which frees dead
	 * inputs and releases successors) runs as soon as the operator is enqueued; only results that land in
	 * host memory (IO nodes such as the logits) are waited for first.
	 */
	void B200Backend::submit(OperatorNode *op_node_ptr, std::function<void()> &&callback) {
		if (submit_planned(op_node_ptr)) {
			if (callback) { callback(); }
			return;
		}
		spyb_op_desc desc{};
		desc.op_type   = static_cast<int32_t>(op_node_ptr->op_type);
		desc.num_input = static_cast<int32_t>(std::min<size_t>(op_node_ptr->num_input(), 3));

		for (int i = 0; i < desc.num_input; ++i) {
			const DataNode *data_node = op_node_ptr->input_data(i);
			void *device_ptr = nullptr;
			if (data_node->node_prop.node_type == DataNodeType::Constant) {
				const Shape &shape = data_node->tensor.get_shape();
				device_ptr = spyb_upload_constant(handle_, data_node->name.c_str(), data_node->tensor.get(),
					static_cast<uint64_t>(data_node->tensor.total_size()), static_cast<int32_t>(shape.number_type), shape.elements.data());
				spy_assert(device_ptr != nullptr, "B200 backend: {}", spyb_last_error(handle_));
			}
			desc.input[i] = to_pod(data_node, device_ptr);
		}
		DataNode *output_node = (op_node_ptr->num_output() > 0) ? op_node_ptr->output_data(0) : nullptr;
		if (output_node != nullptr) { desc.output = to_pod(output_node); }

		switch (op_node_ptr->op_type) {
		case OperatorType::Softmax:
			desc.softmax_scale = static_cast<OperatorDefinition<OperatorType::Softmax> *>(op_node_ptr)->params.get_val().scale; break;
		case OperatorType::NormRMS:
			desc.norm_eps = static_cast<OperatorDefinition<OperatorType::NormRMS> *>(op_node_ptr)->params.get_val().eps; break;
		case OperatorType::View:
			desc.view_offset = static_cast<OperatorDefinition<OperatorType::View> *>(op_node_ptr)->params.get_val().offset; break;
		case OperatorType::Rope: {
			const auto &rope = static_cast<OperatorDefinition<OperatorType::Rope> *>(op_node_ptr)->params.get_val();
			desc.rope = spyb_rope_param{
				static_cast<int32_t>(rope.mode), rope.num_past, rope.num_dim, rope.num_context, rope.num_origin_context,
				rope.freq_base, rope.freq_scale, rope.extend_factor, rope.attention_factor, rope.beta_fast, rope.beta_slow,
				rope.xpos_base, rope.xpos_down ? 1 : 0
			};
		} break;
		default: break;
		}

		const spyb_status status = spyb_submit(handle_, &desc, nullptr, nullptr);
		spy_assert(status == SPYB_SUCCESS, "B200 backend failed on operator {}: {}", op_node_ptr->name, spyb_last_error(handle_));

		// view-type operators (and Copy) report the pointer their output aliases (backend/host/operator/view.cpp:224-276)
		if (output_node != nullptr && is_view(op_node_ptr->op_type)) { output_node->tensor.set_data_ptr(desc.output.data); }
		if (output_node != nullptr && output_node->node_prop.node_type == DataNodeType::IO) {
			spy_assert(spyb_sync(handle_) == SPYB_SUCCESS, "B200 backend: {}", spyb_last_error(handle_));
		}
		if (callback) { callback(); }
	}

	void init_backend(BackendFactory &factory) {
		using BackendConfiguration = BackendFactory::BackendConfiguration;
		const auto generator = +[](const BackendConfiguration &config) -> std::unique_ptr<Backend> {
			return std::make_unique<B200Backend>(config);
		};
		factory.add_backend_map(BackendFactory::make_backend_name("gpu", "b200"), generator);
		factory.add_backend_map(BackendFactory::make_backend_name("gpu", "default"), generator);
	}

} // namespace spy::gpu
