// Host helper: cut tensor lists into multi-tensor launch descriptors (<= MT_MAX tensors each).
#pragma once
#include <torch/extension.h>
#include <functional>
#include <vector>
#include "sg_native.h"

namespace sgb {

inline int dtype_code(const at::Tensor& t) {
    switch (t.scalar_type()) {
        case at::kFloat: return sg::F32;
        case at::kBFloat16: return sg::BF16;
        case at::kHalf: return sg::F16;
        default: TORCH_CHECK(false, "unsupported dtype ", t.scalar_type());
    }
}

// roles[r]: empty, or one tensor per parameter.  packed_off (optional): integer stored in pointer slot 6.
// fn is called once per descriptor.
inline void for_each_launch(const std::vector<std::vector<at::Tensor>>& roles, const std::vector<std::vector<double>>& ts,
                            const std::vector<int64_t>* packed_off, const std::function<void(sg::MTArgs&)>& fn) {
    size_t n = 0;
    for (auto& r : roles)
        if (!r.empty()) { if (n == 0) n = r.size(); TORCH_CHECK(r.size() == n, "role length mismatch"); }
    if (n == 0) return;
    sg::MTArgs a{};
    int t_off = 0, blk_off = 0;
    a.n = 0; a.blk_start[0] = 0;
    auto flush = [&]() {
        if (a.n == 0) return;
        a.t_off = t_off; a.blk_off = blk_off;
        fn(a);
        t_off += a.n; blk_off += a.blk_start[a.n];
        a.n = 0; a.blk_start[0] = 0;
    };
    for (size_t i = 0; i < n; ++i) {
        int64_t numel = -1;
        bool skip = false;
        for (size_t r = 0; r < roles.size(); ++r) {
            if (roles[r].empty()) continue;
            const at::Tensor& t = roles[r][i];
            if (!t.defined()) { skip = true; break; }
            if (numel < 0) numel = t.numel();
            TORCH_CHECK(t.is_contiguous() && t.is_cuda(), "tensors must be contiguous CUDA tensors");
        }
        if (skip || numel < 0) numel = 0;
        const int t = a.n;
        for (int r = 0; r < sg::MT_NP; ++r)
            a.ptr[r][t] = (!skip && (size_t)r < roles.size() && !roles[r].empty() && roles[r][i].defined()) ? roles[r][i].data_ptr() : nullptr;
        if (packed_off) a.ptr[6][t] = reinterpret_cast<void*>(static_cast<intptr_t>((*packed_off)[i]));
        a.numel[t] = numel;
        a.blk_start[t + 1] = a.blk_start[t] + (int)((numel + sg::MT_CHUNK - 1) / sg::MT_CHUNK);
        for (int k = 0; k < sg::MT_NS; ++k) a.ts[t][k] = (i < ts.size() && (size_t)k < ts[i].size()) ? (float)ts[i][k] : 0.f;
        a.n += 1;
        if (a.n == sg::MT_MAX) flush();
    }
    flush();
}

}  // namespace sgb
