// Host-side fast path of the Python operators: the common case of paged_attention_decode, paged_attention_prefill and
// fill_kv_pages - CUDA tensors that are already contiguous and already carry 32-bit (64-bit for slot ids) indices,
// torch's current stream, a workspace that exists - checked and handed to the C ABI (include/pal_b200.h) from C++.
//
// The Python wrappers in ops.py mirror the reference's operator layer (src/proxy_attention_lab/ops.py:33-171,
// src/pal_core/src/ops.cpp:36-239) and do the same through ctypes; a small call spends most of its ~16 us there, in
// attribute reads and argument marshalling.  Every function here returns None when a call is not the common case
// (another dtype, a non-contiguous tensor, an index tensor to convert, no workspace yet, a shape it does not like), and
// the wrapper then takes its usual path, which converts what has to be converted and raises the reference's errors.
// Nothing is computed here, and there is no other route to the GPU than the C ABI.
#include <torch/extension.h>

#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAStream.h>

#include <stdexcept>

#include "pal_b200.h"

namespace {

inline int dtype_code(const at::Tensor& t) {
  if (t.scalar_type() == at::kHalf) return PAL_DTYPE_F16;
  if (t.scalar_type() == at::kBFloat16) return PAL_DTYPE_BF16;
  return -1;
}
inline bool dense_cuda(const at::Tensor& t, const c10::Device& dev) { return t.is_cuda() && t.device() == dev && t.is_contiguous(); }
inline bool int32_like(const at::Tensor& t) { return t.scalar_type() == at::kInt || t.scalar_type() == at::kUInt32; }

void raise_for(int rc) {
  if (rc == PAL_OK) return;
  const char* msg = pal_last_error();
  std::string text = (msg && *msg) ? msg : ("pal_b200 error " + std::to_string(rc));
  if (rc == PAL_ERR_BAD_ARG) throw py::value_error(text);
  throw std::runtime_error(text);
}

// The newest workspace the Python layer holds for (device, stream), if it has `need` bytes; nullptr otherwise.
// `registry` is ops._WORKSPACES: {(device index, cudaStream_t as int): [tensor, ...]}.
void* held_workspace(const py::dict& registry, int device_index, cudaStream_t stream, size_t need, size_t* bytes) {
  py::tuple key = py::make_tuple(device_index, reinterpret_cast<uintptr_t>(stream));
  PyObject* held = PyDict_GetItem(registry.ptr(), key.ptr());  // borrowed
  if (!held || !PyList_Check(held) || PyList_GET_SIZE(held) == 0) return nullptr;
  PyObject* last = PyList_GET_ITEM(held, PyList_GET_SIZE(held) - 1);
  if (!THPVariable_Check(last)) return nullptr;
  const at::Tensor& ws = THPVariable_Unpack(last);
  if ((size_t)ws.numel() < need) return nullptr;
  *bytes = (size_t)ws.numel();
  return ws.data_ptr();
}

// paged_attention_decode / paged_attention_decode_append (new_k, new_v given)
py::object decode(const at::Tensor& q, const at::Tensor& k_pool, const at::Tensor& v_pool, const at::Tensor& page_table,
                  const at::Tensor& seq_lens, int partition_pages, double scale, bool out_f32, const py::dict& registry,
                  const c10::optional<at::Tensor>& new_k, const c10::optional<at::Tensor>& new_v) {
  if (!q.is_cuda()) return py::none();
  const c10::Device dev = q.device();
  const int code = dtype_code(q);
  if (code < 0 || v_pool.dim() != 4 || k_pool.dim() != 5 || page_table.dim() != 2 || q.dim() != 3) return py::none();
  if (!dense_cuda(q, dev) || !dense_cuda(k_pool, dev) || !dense_cuda(v_pool, dev) || !dense_cuda(page_table, dev) ||
      !dense_cuda(seq_lens, dev) || !int32_like(page_table) || !int32_like(seq_lens) || k_pool.scalar_type() != q.scalar_type() ||
      v_pool.scalar_type() != q.scalar_type())
    return py::none();
  const int64_t num_pages = v_pool.size(0), hkv = v_pool.size(1), d = v_pool.size(2), tpp = v_pool.size(3);
  const int64_t S = page_table.size(0), mp = page_table.size(1), hq = q.size(1);
  if (S == 0 || mp == 0 || num_pages == 0 || hkv == 0 || q.size(0) < S || q.size(2) != d || seq_lens.numel() < S || hq % hkv != 0 ||
      k_pool.size(0) != num_pages || k_pool.size(1) != hkv || k_pool.size(2) * 8 != d || k_pool.size(3) != tpp || k_pool.size(4) != 8)
    return py::none();
  const bool append = new_k.has_value();
  if (append) {
    if (!new_v.has_value()) return py::none();
    for (const at::Tensor* t : {&*new_k, &*new_v})
      if (!dense_cuda(*t, dev) || t->scalar_type() != q.scalar_type() || t->dim() != 3 || t->size(0) != S || t->size(1) != hkv || t->size(2) != d)
        return py::none();
  }
  c10::cuda::CUDAGuard guard(dev);
  const cudaStream_t stream = c10::cuda::getCurrentCUDAStream(dev.index()).stream();
  const size_t need = pal_decode_workspace_bytes((int)S, (int)hq, (int)hkv, (int)d, (int)tpp, (int)mp, partition_pages);
  size_t ws_bytes = 0;
  void* ws = held_workspace(registry, dev.index(), stream, need > 256 ? need : 256, &ws_bytes);
  if (!ws) return py::none();
  at::Tensor out = at::empty({S, hq, d}, q.options().dtype(out_f32 ? at::kFloat : q.scalar_type()));
  const int dt = code | (out_f32 ? PAL_OUT_F32 : 0);
  int rc;
  if (append)
    rc = pal_paged_attention_decode_append(new_k->data_ptr(), new_v->data_ptr(), q.data_ptr(), k_pool.data_ptr(), v_pool.data_ptr(),
                                           page_table.data_ptr(), static_cast<const int32_t*>(seq_lens.data_ptr()), out.data_ptr(), (int)S,
                                           (int)hq, (int)hkv, (int)d, (int)tpp, num_pages, (int)mp, (float)scale, dt, partition_pages, ws,
                                           ws_bytes, stream);
  else
    rc = pal_paged_attention_decode(q.data_ptr(), k_pool.data_ptr(), v_pool.data_ptr(), page_table.data_ptr(),
                                    static_cast<const int32_t*>(seq_lens.data_ptr()), out.data_ptr(), (int)S, (int)hq, (int)hkv, (int)d,
                                    (int)tpp, num_pages, (int)mp, (float)scale, dt, partition_pages, ws, ws_bytes, stream);
  raise_for(rc);
  return py::cast(out);
}

// paged_attention_prefill (uniform batches) / paged_attention_prefill_ragged (cu_seqlens and the longest count given)
py::object prefill(const at::Tensor& q, const at::Tensor& k, const at::Tensor& v, const at::Tensor& k_pool, const at::Tensor& v_pool,
                   const at::Tensor& page_table, const at::Tensor& hist, int impl, double scale, bool out_f32, const py::dict& registry,
                   const c10::optional<at::Tensor>& cu_seqlens, int max_new_tokens) {
  if (!q.is_cuda()) return py::none();
  const c10::Device dev = q.device();
  const int code = dtype_code(q);
  if (code < 0 || v_pool.dim() != 4 || k_pool.dim() != 5 || page_table.dim() != 2 || q.dim() != 3 || k.dim() != 3 || v.dim() != 3)
    return py::none();
  for (const at::Tensor* t : {&q, &k, &v, &k_pool, &v_pool})
    if (!dense_cuda(*t, dev) || t->scalar_type() != q.scalar_type()) return py::none();
  if (!dense_cuda(page_table, dev) || !dense_cuda(hist, dev) || !int32_like(page_table) || !int32_like(hist)) return py::none();
  const int64_t num_pages = v_pool.size(0), hkv = v_pool.size(1), d = v_pool.size(2), tpp = v_pool.size(3);
  const int64_t S = page_table.size(0), mp = page_table.size(1), total = q.size(0), hq = q.size(1);
  const bool ragged = cu_seqlens.has_value();
  if (ragged && (!dense_cuda(*cu_seqlens, dev) || !int32_like(*cu_seqlens) || cu_seqlens->dim() != 1 || cu_seqlens->numel() != S + 1 ||
                 max_new_tokens <= 0))
    return py::none();
  if (S == 0 || total == 0 || (!ragged && total % S != 0) || num_pages == 0 || mp == 0 || hkv == 0 || hq % hkv != 0 || q.size(2) != d ||
      k.size(0) != total || v.size(0) != total || k.size(1) != hkv || v.size(1) != hkv || k.size(2) != d || v.size(2) != d ||
      hist.numel() < S || k_pool.size(0) != num_pages || k_pool.size(1) != hkv || k_pool.size(2) * 8 != d || k_pool.size(3) != tpp ||
      k_pool.size(4) != 8)
    return py::none();
  c10::cuda::CUDAGuard guard(dev);
  const cudaStream_t stream = c10::cuda::getCurrentCUDAStream(dev.index()).stream();
  size_t ws_bytes = 0;
  const int per_seq = ragged ? max_new_tokens : (int)(total / S);
  const size_t need = pal_prefill_workspace_bytes((int)S, per_seq, (int)hq, (int)hkv, (int)d);
  void* ws = held_workspace(registry, dev.index(), stream, need > 256 ? need : 256, &ws_bytes);
  if (!ws) return py::none();
  at::Tensor out = at::empty({total * hq, d}, q.options().dtype(out_f32 ? at::kFloat : q.scalar_type()));
  const int dt = code | (out_f32 ? PAL_OUT_F32 : 0);
  int rc;
  if (ragged)
    rc = pal_paged_attention_prefill_ragged(q.data_ptr(), k.data_ptr(), v.data_ptr(), k_pool.data_ptr(), v_pool.data_ptr(), page_table.data_ptr(),
                                            static_cast<const int32_t*>(hist.data_ptr()), static_cast<const int32_t*>(cu_seqlens->data_ptr()),
                                            out.data_ptr(), (int)S, total, max_new_tokens, (int)hq, (int)hkv, (int)d, (int)tpp, num_pages,
                                            (int)mp, (float)scale, dt, impl, ws, ws_bytes, stream);
  else
    rc = pal_paged_attention_prefill(q.data_ptr(), k.data_ptr(), v.data_ptr(), k_pool.data_ptr(), v_pool.data_ptr(), page_table.data_ptr(),
                                     static_cast<const int32_t*>(hist.data_ptr()), out.data_ptr(), (int)S, per_seq, (int)hq, (int)hkv, (int)d,
                                     (int)tpp, num_pages, (int)mp, (float)scale, dt, impl, ws, ws_bytes, stream);
  raise_for(rc);
  return py::cast(out);
}

// fill_kv_pages, in place; `a` is the slot mapping (int64) when `pos` and `seq_map` are None, else the page table.
// Returns True when the call was made.
bool fill(const at::Tensor& new_k, const at::Tensor& new_v, const at::Tensor& k_pool, const at::Tensor& v_pool, const at::Tensor& a,
          const c10::optional<at::Tensor>& pos, const c10::optional<at::Tensor>& seq_map) {
  if (!v_pool.is_cuda()) return false;
  const c10::Device dev = v_pool.device();
  const int code = dtype_code(v_pool);
  if (code < 0 || v_pool.dim() != 4 || k_pool.dim() != 5 || new_k.dim() != 3 || new_v.dim() != 3) return false;
  for (const at::Tensor* t : {&new_k, &new_v, &k_pool, &v_pool})
    if (!dense_cuda(*t, dev) || t->scalar_type() != v_pool.scalar_type()) return false;
  const int64_t num_pages = v_pool.size(0), hkv = v_pool.size(1), d = v_pool.size(2), tpp = v_pool.size(3), T = new_k.size(0);
  if (T == 0 || num_pages == 0 || new_k.size(1) != hkv || new_k.size(2) != d || new_v.size(0) != T || new_v.size(1) != hkv ||
      new_v.size(2) != d || k_pool.size(0) != num_pages || k_pool.size(1) != hkv || k_pool.size(2) * 8 != d || k_pool.size(3) != tpp ||
      k_pool.size(4) != 8 || !dense_cuda(a, dev))
    return false;
  c10::cuda::CUDAGuard guard(dev);
  const cudaStream_t stream = c10::cuda::getCurrentCUDAStream(dev.index()).stream();
  int rc;
  if (!pos.has_value()) {
    if (seq_map.has_value() || a.scalar_type() != at::kLong || a.numel() != T) return false;
    rc = pal_fill_kv_pages_slots(new_k.data_ptr(), new_v.data_ptr(), k_pool.data_ptr(), v_pool.data_ptr(),
                                 static_cast<const int64_t*>(a.data_ptr()), T, (int)hkv, (int)d, (int)tpp, num_pages, code, stream);
  } else {
    if (!seq_map.has_value() || a.dim() != 2 || !int32_like(a) || !dense_cuda(*pos, dev) || !dense_cuda(*seq_map, dev) || !int32_like(*pos) ||
        !int32_like(*seq_map) || pos->numel() != T || seq_map->numel() != T)
      return false;
    rc = pal_fill_kv_pages(new_k.data_ptr(), new_v.data_ptr(), k_pool.data_ptr(), v_pool.data_ptr(), a.data_ptr(),
                           static_cast<const int32_t*>(pos->data_ptr()), seq_map->data_ptr(), T, (int)a.size(0), (int)hkv, (int)d, (int)tpp,
                           num_pages, (int)a.size(1), code, stream);
  }
  raise_for(rc);
  return true;
}

}  // namespace

PYBIND11_MODULE(_pal_fast, m) {
  m.doc() = "C++ fast path of the pal_b200 Python operators (argument checks and the C-ABI call without ctypes)";
  m.def("decode", &decode);
  m.def("prefill", &prefill);
  m.def("fill", &fill);
}
