/*
 * Body fragment for RegionLayer<Device::CUDA>::addDetects(Detections& detects, int width, int height, float threshold),
 * replacing include/cuda/RegionLayer.h:76-82 (the whole output copied to the host, then the loops of
 * include/RegionLayer.h:355-381 once per image).  per_image = 0 keeps the reference's indexing: its helper reads the
 * predictions without the image's offset (include/RegionLayer.h:363-369), so every image decodes image 0's boxes;
 * pass 1 to give each image its own.
 *
 * Uses the reference's members output_, batch(), width(), height(), classes(), num_, coords_, anchors_
 * (std::vector<float>, 2 * num_ values); added by the integration: pxeDets_ (PxCudaVectorT<char>, capacity
 * pxeCapacity_ records of 32 bytes) and pxeCount_ (PxCudaVectorT<long long>, 1 element), allocated once in setup().
 */
{
    long long zero = 0;
    PX_CUDA_CHECK_ERR(cudaMemcpy(pxeCount_.data(), &zero, sizeof zero, cudaMemcpyHostToDevice));
    PXE_CHECK(pxe_region_decode(nullptr, this->output_.data(), this->batch(), this->width(), this->height(), num_, coords_,
                                this->classes(), anchors_.data(), /*per_image=*/0, (float)width, (float)height, threshold,
                                reinterpret_cast<pxe_detection*>(pxeDets_.data()), pxeCapacity_, pxeCount_.data(), 0));
    long long total = 0;
    PX_CUDA_CHECK_ERR(cudaMemcpy(&total, pxeCount_.data(), sizeof total, cudaMemcpyDeviceToHost));
    const long long n = total < pxeCapacity_ ? total : pxeCapacity_;
    std::vector<pxe_detection> host((size_t)n);
    PX_CUDA_CHECK_ERR(cudaMemcpy(host.data(), pxeDets_.data(), (size_t)n * sizeof(pxe_detection), cudaMemcpyDeviceToHost));
    for (const pxe_detection& r : host)
        detects.emplace_back(cv::Rect2f(r.x, r.y, r.w, r.h), r.batch_id, r.class_id, r.prob);
}
