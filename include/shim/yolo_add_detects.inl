/*
 * Body fragment for YoloLayer<Device::CUDA>::addDetects(Detections& detects, int width, int height, float threshold)
 * (and, with width = height = 0, for the overload without an image size), replacing the whole-head device-to-host copy
 * and the host loops of include/cuda/YoloLayer.h:168-188 -> include/YoloLayer.h:659-698.
 *
 * Uses the reference's members output_, batch(), outHeight(), outWidth(), mask_, anchors_, classes(), model();
 * added by the integration: pxeDets_ (PxCudaVectorT<char>, capacity pxeCapacity_ records of 32 bytes),
 * pxeCount_ (PxCudaVectorT<long long>, 1 element), pxeWorkspace_ (PxCudaVectorT<char>, sized in setup() with
 * pxe_yolo_decode_workspace_bytes), all allocated once in setup().
 */
{
    pxe_yolo_decode_desc d{};
    d.head = this->output_.data();                 /* activated by YoloLayer<CUDA>::forward */
    d.batch = this->batch();
    d.height = this->outHeight();
    d.width = this->outWidth();
    d.classes = this->classes();
    d.n_masks = (int)mask_.size();
    for (int i = 0; i < d.n_masks; ++i) d.mask[i] = mask_[i];
    d.n_anchor_values = (int)anchors_.size();
    for (int i = 0; i < d.n_anchor_values; ++i) d.anchors[i] = anchors_[i];
    d.net_width = this->model().width();
    d.net_height = this->model().height();
    d.image_width = width;
    d.image_height = height;
    d.threshold = threshold;
    long long zero = 0;
    PX_CUDA_CHECK_ERR(cudaMemcpy(pxeCount_.data(), &zero, sizeof zero, cudaMemcpyHostToDevice));
    PXE_CHECK(pxe_yolo_decode(nullptr, &d, reinterpret_cast<pxe_detection*>(pxeDets_.data()), pxeCapacity_,
                              pxeCount_.data(), pxeWorkspace_.data(), pxeWorkspace_.size()));
    long long total = 0;
    PX_CUDA_CHECK_ERR(cudaMemcpy(&total, pxeCount_.data(), sizeof total, cudaMemcpyDeviceToHost));
    const long long n = total < pxeCapacity_ ? total : pxeCapacity_;
    std::vector<pxe_detection> host((size_t)n);
    PX_CUDA_CHECK_ERR(cudaMemcpy(host.data(), pxeDets_.data(), (size_t)n * sizeof(pxe_detection), cudaMemcpyDeviceToHost));
    for (const pxe_detection& r : host)
        detects.emplace_back(cv::Rect2f(r.x, r.y, r.w, r.h), r.batch_id, r.class_id, r.prob);
}
