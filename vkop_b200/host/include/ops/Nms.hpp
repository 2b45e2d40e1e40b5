// NMS operator: interface of the reference's ops/Nms.hpp (:28-115).
// Attributes "center_point_box" (0), "iou_threshold" (0), "score_threshold"
// (0), "max_output_boxes_per_class" (0 = unlimited), as the reference, plus
// "pre_topk" (0): only the best pre_topk candidates of a class enter the sweep.
// Inputs: boxes [B, N, 4] and scores [B, C, N], fp32 -- or one detection head
// [B, 4 + C, N] (coordinate planes, then score planes), used in place.  Output: int rows
// (batch, class, box).  Differences from the reference (its shader writes rows
// at atomically claimed offsets, sizes the output without the batch factor and
// never clears its counter, ops/Nms.hpp:79-86,105-106): rows come in
// (batch, class, rank) order, an empty output is sized for every batch
// (B * C * per-class bound rows), rows past the result are filled with -1,
// and the number of rows is available from last_count() after the work is done.
#ifndef VKOP_HOST_OPS_NMS_HPP_
#define VKOP_HOST_OPS_NMS_HPP_

#include "ops/Operator.hpp"

namespace vkop {
namespace ops {

class Nms : public Operator {
  public:
    Nms() : Operator(OpType::NMS) {}

    void setAttribute(const std::unordered_map<std::string, std::string> &attributes) override {
        if (attributes.count("center_point_box"))
            center_point_box_ = static_cast<int>(std::stol(attributes.at("center_point_box")));
        if (attributes.count("iou_threshold"))
            iou_threshold_ = std::stof(attributes.at("iou_threshold"));
        if (attributes.count("score_threshold"))
            score_threshold_ = std::stof(attributes.at("score_threshold"));
        if (attributes.count("max_output_boxes_per_class"))
            max_output_boxes_per_class_ = static_cast<int>(std::stol(attributes.at("max_output_boxes_per_class")));
        if (attributes.count("pre_topk"))
            pre_topk_ = static_cast<int>(std::stol(attributes.at("pre_topk")));
    }

    // Rows produced by the last execution; waits for that execution to finish.
    int last_count() {
        if (!count_)
            return 0;
        m_cmd_->wait();
        int32_t n = 0;
        cuda_check(cudaMemcpy(&n, count_->ptr(), sizeof(n), cudaMemcpyDeviceToHost), "cudaMemcpy count");
        return n;
    }

  private:
    void execute(const std::vector<std::shared_ptr<core::ITensor>> &inputs,
                 const std::vector<std::shared_ptr<core::ITensor>> &outputs) override {
        // One input: a detection head [B, 4 + C, N] (coordinate planes, then class-score planes), used in
        // place.  Two inputs: boxes [B, N, 4] and scores [B, C, N] as in the reference.
        const bool head = inputs.size() == 1;
        int batch, num_boxes, num_class;
        if (head) {
            const auto shape = inputs[0]->getShape();
            if (shape.size() != 3 || shape[1] <= 4)
                throw std::invalid_argument("Nms: a single input must be a detection head [B, 4 + C, N]");
            if (inputs[0]->dtype() != typeid(float))
                throw std::invalid_argument("Nms: the detection head must be a float tensor");
            batch = shape[0];
            num_class = shape[1] - 4;
            num_boxes = shape[2];
        } else {
            const auto box_shape = inputs[0]->getShape();
            const auto score_shape = inputs[1]->getShape();
            if (box_shape.size() != 3 || score_shape.size() != 3 || box_shape[2] != 4)
                throw std::invalid_argument("Nms: boxes must be [B, N, 4] and scores [B, C, N]");  // the reference asserts
            if (inputs[0]->dtype() != typeid(float) || inputs[1]->dtype() != typeid(float))
                throw std::invalid_argument("Nms: boxes and scores must be float tensors");
            batch = box_shape[0];
            num_boxes = box_shape[1];
            num_class = score_shape[1];
            if (score_shape[0] != batch || score_shape[2] != num_boxes)
                throw std::invalid_argument("Nms: boxes and scores disagree on batch or box count");
        }
        if (outputs[0]->dtype() != typeid(int))
            throw std::invalid_argument("Nms: the output must be an int tensor");
        int per_class = num_boxes;
        if (pre_topk_ > 0 && pre_topk_ < per_class)
            per_class = pre_topk_;
        if (max_output_boxes_per_class_ > 0 && max_output_boxes_per_class_ < per_class)
            per_class = max_output_boxes_per_class_;
        resize_if_empty(outputs[0], std::vector<int>{batch * num_class * per_class, 3});
        vkop_nms_desc d;
        d.num_batch = batch;
        d.num_class = num_class;
        d.num_boxes = num_boxes;
        d.center_point_box = center_point_box_;
        d.max_output_boxes_per_class = max_output_boxes_per_class_;
        d.pre_topk = pre_topk_;
        d.iou_threshold = iou_threshold_;
        d.score_threshold = score_threshold_;
        d.capacity_rows = outputs[0]->num_elements() / 3;
        size_t need = 0;
        check(vkop_cuda_nms_workspace(&d, &need), "vkop_cuda_nms_workspace");
        void *ws = workspace(need);
        if (!count_)
            count_ = std::make_shared<core::DeviceBuffer>(16);
        void *out = device_of(outputs[0]);
        cuda_check(cudaMemsetAsync(out, 0xFF, static_cast<size_t>(outputs[0]->num_elements()) * sizeof(int), stream()),
                   "cudaMemsetAsync");  // rows past the result read (-1, -1, -1)
        if (head)
            check(vkop_cuda_yolo_nms(&d, device_of(inputs[0]), static_cast<int32_t *>(out), static_cast<int32_t *>(count_->ptr()),
                                     ws, workspace_bytes(), stream()),
                  "vkop_cuda_yolo_nms");
        else
            check(vkop_cuda_nms(&d, device_of(inputs[0]), device_of(inputs[1]), static_cast<int32_t *>(out),
                                static_cast<int32_t *>(count_->ptr()), ws, workspace_bytes(), stream()),
                  "vkop_cuda_nms");
    }

    int center_point_box_ = 0, max_output_boxes_per_class_ = 0, pre_topk_ = 0;
    float iou_threshold_ = 0.0f, score_threshold_ = 0.0f;
    std::shared_ptr<core::DeviceBuffer> count_;
};

}  // namespace ops
}  // namespace vkop
#endif  // VKOP_HOST_OPS_NMS_HPP_
