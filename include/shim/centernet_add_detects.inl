/*
 * Body fragment for CenterNetLayer<Device::CUDA>::addDetects(Detections& detections, int width, int height,
 * float threshold) (width = height = 0 for the overload without an image size), replacing the whole-tensor
 * device-to-host copy and the host loops of include/cuda/CenterNetLayer.h:89-106 -> include/CenterNetLayer.h:196-247.
 *
 * Uses the reference's members output_ (activated by forward), batch(), outputs(), outHeight(), outWidth(), classes_,
 * maxDetections_; added by the integration: pxeDets_ (batch() * maxDetections_ records of 32 bytes), pxeCounts_
 * (batch() ints), pxeWorkspace_ (pxe_centernet_decode_workspace_bytes), allocated once in setup().
 */
{
    const long long area = (long long)this->outHeight() * this->outWidth();
    pxe_centernet_decode_desc d{};
    d.heat = this->output_.data();
    d.heat_batch_stride = this->outputs();
    d.size = this->output_.data() + (long long)classes_ * area;
    d.size_batch_stride = this->outputs();
    d.offset = this->output_.data() + (long long)(classes_ + 2) * area;
    d.offset_batch_stride = this->outputs();
    d.heat_is_logit = 0;                           /* output_ holds the activated scores */
    d.batch = this->batch();
    d.classes = classes_;
    d.height = this->outHeight();
    d.width = this->outWidth();
    d.image_width = width;
    d.image_height = height;
    d.threshold = threshold;
    d.max_detections = maxDetections_;
    PXE_CHECK(pxe_centernet_decode(nullptr, &d, reinterpret_cast<pxe_detection*>(pxeDets_.data()), pxeCounts_.data(),
                                   pxeWorkspace_.data(), pxeWorkspace_.size()));
    std::vector<int> counts((size_t)this->batch());
    PX_CUDA_CHECK_ERR(cudaMemcpy(counts.data(), pxeCounts_.data(), counts.size() * sizeof(int), cudaMemcpyDeviceToHost));
    std::vector<pxe_detection> host((size_t)this->batch() * maxDetections_);
    PX_CUDA_CHECK_ERR(cudaMemcpy(host.data(), pxeDets_.data(), host.size() * sizeof(pxe_detection), cudaMemcpyDeviceToHost));
    for (int b = 0; b < this->batch(); ++b)
        for (int i = 0; i < counts[(size_t)b]; ++i) {
            const pxe_detection& r = host[(size_t)b * maxDetections_ + i];
            detections.emplace_back(cv::Rect2f(r.x, r.y, r.w, r.h), r.batch_id, r.class_id, r.prob);
        }
}
