/*
 * Body fragment for DetectLayer<Device::CUDA>::addDetects(Detections& detects, int width, int height, float threshold)
 * (the YOLOv1 head), replacing include/cuda/DetectLayer.h:81-86: the whole head copied to the host, then the loops of
 * include/DetectLayer.h:166-209 per image.  The decode runs on the layer's device output; only the boxes it emits
 * come back.
 *
 * Uses the reference's members output_, batch(), outputs(), classes(), side_, num_, coords_, sqrt_; added by the
 * integration: pxeDets_ (PxCudaVectorT<char>, capacity pxeCapacity_ records of 32 bytes; batch() * side_ * side_ *
 * num_ records always suffice) and pxeCount_ (PxCudaVectorT<long long>, 1 element), allocated once in setup().
 */
{
    long long zero = 0;
    PX_CUDA_CHECK_ERR(cudaMemcpy(pxeCount_.data(), &zero, sizeof zero, cudaMemcpyHostToDevice));
    PXE_CHECK(pxe_detect_decode(nullptr, this->output_.data(), this->outputs(), this->batch(), side_, num_, this->classes(),
                                coords_, sqrt_ ? 1 : 0, (float)width, (float)height, threshold,
                                reinterpret_cast<pxe_detection*>(pxeDets_.data()), pxeCapacity_, pxeCount_.data(), 0));
    long long total = 0;
    PX_CUDA_CHECK_ERR(cudaMemcpy(&total, pxeCount_.data(), sizeof total, cudaMemcpyDeviceToHost));
    const long long n = total < pxeCapacity_ ? total : pxeCapacity_;
    std::vector<pxe_detection> host((size_t)n);
    PX_CUDA_CHECK_ERR(cudaMemcpy(host.data(), pxeDets_.data(), (size_t)n * sizeof(pxe_detection), cudaMemcpyDeviceToHost));
    for (const pxe_detection& r : host)
        detects.emplace_back(cv::Rect2f(r.x, r.y, r.w, r.h), r.batch_id, r.class_id, r.prob);
}
