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
	}

	B200Backend::~B200Backend() noexcept { spyb_destroy(handle_); }

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
