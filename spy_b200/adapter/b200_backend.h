// spy::Backend implementation over the C ABI of libspyb200.so.
//
// This is the only translation unit family that includes the reference's headers: it turns each
// OperatorNode the reference's scheduler submits into the plain-C spyb_op_desc and forwards it.
// Registration follows the hook the reference already has for a CUDA backend
// (backend/interface/include/backend/backend.h:142-155, backend/cuda/backend/cuda.cu:10-21):
// compile the reference with -DSPY_BACKEND_CUDA and link this file, and
// BackendFactory::init_backend("gpu:b200", config) (or the reference CLI's "gpu:default") yields it.
#pragma once

#include <memory>
#include <mutex>
#include <string>
#include <unordered_map>

#include "backend/backend.h"
#include "graph/graph.h"
#include "operator/operator.h"

#include "../../include/spyb.h"

namespace spy::gpu {

	class B200Backend final: public Backend {
	private:
		spyb_backend *handle_ = nullptr;
		int           device_id_ = 0;

		// Plan mode (configuration key "model" = path of the GGUF file the graph was built from): the steps of the LLaMa
		// graph are served from the library's fused step plan instead of operator by operator. The scheduler still walks
		// its graph and submits every node; the adapter only notes the step's inputs (token ids from the embedding
		// GetRow, the position from the first Rope), keeps the pointer aliasing of view-type operators alive, and runs
		// the whole step when the node that produces the logits arrives.
		std::string     plan_path_;
		int             plan_context_ = 512;
		bool            plan_enabled_ = false, plan_tried_ = false;
		spyb_model     *plan_model_ = nullptr;
		const int32_t  *plan_ids_ = nullptr;
		int             plan_num_token_ = 0, plan_num_past_ = -1;

	public:
		explicit B200Backend(const BackendFactory::BackendConfiguration &config);

		~B200Backend() noexcept override;

	public:
		size_t get_max_memory_capacity()   const override { return spyb_max_memory(handle_); }
		size_t get_avail_memory_capacity() const override { return spyb_avail_memory(handle_); }

		void *alloc_memory(size_t size) override;
		void  dealloc_memory(void *ptr, size_t size) override { spyb_free(handle_, ptr, size); }

		size_t get_max_concurrency()   const override { return 1; }
		size_t get_avail_concurrency() const override { return 1; }

		bool is_support(OperatorType op_type) const override { return spyb_is_support(static_cast<int32_t>(op_type)) != 0; }

		void submit(OperatorNode *op_node_ptr, std::function<void()> &&callback = nullptr) override;

	public:
		spyb_backend *handle() const { return handle_; }
		bool plan_active() const { return plan_model_ != nullptr; }

	private:
		bool submit_planned(OperatorNode *op_node_ptr);
	};

	void init_backend(BackendFactory &factory);

} // namespace spy::gpu
