"""Launch wrappers over the C ABI -- the counterpart of the reference's ``khq_*_try_launch``
functions (``src/ops.mojo:1101-1279``), taking torch CUDA tensors instead of raw pointers.

Differences from the reference wrappers: the library is loaded once (the reference re-opens it
and re-reads ``BONSAI_DISABLE_CUDA_FFI`` on every call), launches go to torch's current stream
(the reference passes a NULL stream), and a non-zero return raises instead of returning False.
"""
from __future__ import annotations

from . import lib as _lib
from .lib import check, current_stream, ptr


class CudaOps:
    """The product's only compute backend: every method is one call into the CUDA library."""

    name = "cuda"

    def __init__(self):
        self.lib = _lib.load()

    # -- launch_khq_compress_fp16 ------------------------------------------------------------
    def compress(self, x, d_vec, rotor, centroids, vq_centroids, out_mask, out_norms, out_r_norms,
                 out_payload, out_shared_meta, n, d, ts, alpha, is_v):
        rc = self.lib.launch_khq_compress_fp16(
            ptr(x), ptr(d_vec), ptr(rotor), ptr(centroids), ptr(vq_centroids), ptr(out_mask),
            ptr(out_norms), ptr(out_r_norms), ptr(out_payload), ptr(out_shared_meta), int(n),
            int(d), float(ts), float(alpha), 1 if is_v else 0, current_stream())
        check("launch_khq_compress_fp16", rc)

    # -- launch_khq_attn_fp16 ----------------------------------------------------------------
    def attn(self, q, k_payload, v_payload, v_shared_meta, k_mask, k_norms, k_r_norms, v_norms,
             v_r_norms, centroids_k, centroids_v, vq_centroids, k_rotor, v_rotor, d_vec_k, d_vec_v,
             out_attn, out_partial, num_queries, num_heads, L_q, c_len, stride_s, n_rep, scale,
             alpha_k, alpha_v, rope_base, start_pos, num_splits):
        rc = self.lib.launch_khq_attn_fp16(
            ptr(q), ptr(k_payload), ptr(v_payload), ptr(v_shared_meta), ptr(k_mask), ptr(k_norms),
            ptr(k_r_norms), ptr(v_norms), ptr(v_r_norms), ptr(centroids_k), ptr(centroids_v),
            ptr(vq_centroids), ptr(k_rotor), ptr(v_rotor), ptr(d_vec_k), ptr(d_vec_v),
            ptr(out_attn), ptr(out_partial), int(num_queries), int(num_heads), int(L_q),
            int(c_len), int(stride_s), int(n_rep), float(scale), float(alpha_k), float(alpha_v),
            float(rope_base), int(start_pos), int(num_splits), current_stream())
        check("launch_khq_attn_fp16", rc)

    # -- launch_khq_attn_strided_fp16: a slice holding every G-th chunk of a longer context ------------
    def attn_strided(self, q, k_payload, v_payload, v_shared_meta, k_mask, k_norms, k_r_norms, v_norms,
                     v_r_norms, centroids_k, centroids_v, vq_centroids, k_rotor, v_rotor, d_vec_k, d_vec_v,
                     out_attn, out_partial, num_queries, num_heads, L_q, c_len, n_rep, scale, alpha_k, alpha_v,
                     rope_base, start_pos, num_splits, pos_chunk, pos_stride):
        rc = self.lib.launch_khq_attn_strided_fp16(
            ptr(q), ptr(k_payload), ptr(v_payload), ptr(v_shared_meta), ptr(k_mask), ptr(k_norms),
            ptr(k_r_norms), ptr(v_norms), ptr(v_r_norms), ptr(centroids_k), ptr(centroids_v),
            ptr(vq_centroids), ptr(k_rotor), ptr(v_rotor), ptr(d_vec_k), ptr(d_vec_v),
            ptr(out_attn), ptr(out_partial), int(num_queries), int(num_heads), int(L_q), int(c_len),
            int(n_rep), float(scale), float(alpha_k), float(alpha_v), float(rope_base), int(start_pos),
            int(num_splits), int(pos_chunk), int(pos_stride), current_stream())
        check("launch_khq_attn_strided_fp16", rc)

    # -- launch_khq_window_attn_fp16 -----------------------------------------------------------
    def window_attn(self, q, ring_k, ring_v, out_attn, win_start, win_len, ring_cap, H_q, H_kv, d,
                    scale):
        rc = self.lib.launch_khq_window_attn_fp16(
            ptr(q), ptr(ring_k), ptr(ring_v), ptr(out_attn), int(win_start), int(win_len),
            int(ring_cap), int(H_q), int(H_kv), int(d), float(scale), current_stream())
        check("launch_khq_window_attn_fp16", rc)

    # -- launch_khq_merge_gate_fp16, with the argument selection of khq_merge_gate_try
    #    (src/ops.mojo:1255-1279): window only -> attn_c := attn_w and has_w = 0 ----------------
    def merge_gate(self, attn_c, attn_w, q_gate, out, H_q, d, has_w, has_c):
        src_c = attn_c if has_c else attn_w
        rc = self.lib.launch_khq_merge_gate_fp16(
            ptr(src_c), ptr(attn_w), ptr(q_gate), ptr(out), int(H_q), int(d),
            1 if (has_w and has_c) else 0, current_stream())
        check("launch_khq_merge_gate_fp16", rc)

    # -- launch_khq_merge_slots_gate_fp16: finish a context-parallel step ------------------------
    def merge_slots_gate(self, partials, n_slots, q_gate, out, H_q, d):
        rc = self.lib.launch_khq_merge_slots_gate_fp16(ptr(partials), int(n_slots), ptr(q_gate), ptr(out),
                                                       int(H_q), int(d), current_stream())
        check("launch_khq_merge_slots_gate_fp16", rc)

    # -- launch_khq_decode_step_fp16: ring appends + both regions + merge + gate, one call ----------
    def decode_step(self, q_gate, k_roped, v_new, k_unroped, ring_k, ring_v, ring_u, kv, tables, attn_c, attn_partial, out,
                    c_len, win_start, win_len, ring_cap, num_splits, scale, alpha_k, alpha_v, rope_base):
        """kv: dict of the eight payload arrays (k_payload, v_payload, v_shared_meta, k_mask, k_norms,
        k_r_norms, v_norms, v_r_norms); tables: dict (cents_k, cents_v, vq, rotor_k, rotor_v, d_k, d_v)."""
        rc = self.lib.launch_khq_decode_step_fp16(
            ptr(q_gate), ptr(k_roped), ptr(v_new), ptr(k_unroped), ptr(ring_k), ptr(ring_v), ptr(ring_u),
            ptr(kv["k_payload"]), ptr(kv["v_payload"]), ptr(kv["v_shared_meta"]), ptr(kv["k_mask"]), ptr(kv["k_norms"]),
            ptr(kv["k_r_norms"]), ptr(kv["v_norms"]), ptr(kv["v_r_norms"]), ptr(tables["cents_k"]), ptr(tables["cents_v"]),
            ptr(tables["vq"]), ptr(tables["rotor_k"]), ptr(tables["rotor_v"]), ptr(tables["d_k"]), ptr(tables["d_v"]),
            ptr(attn_c), ptr(attn_partial), ptr(out), int(c_len), int(win_start), int(win_len), int(ring_cap),
            int(num_splits), float(scale), float(alpha_k), float(alpha_v), float(rope_base), current_stream())
        check("launch_khq_decode_step_fp16", rc)

    # -- peer-memory exchange of context-parallel partials ----------------------------------------
    def publish_partials(self, src, n_records, peer_slots, peer_flags, world, rank, first_slot, parity_offset_records, epoch):
        rc = self.lib.launch_khq_publish_partials_fp32(ptr(src), int(n_records), ptr(peer_slots), ptr(peer_flags), int(world),
                                                       int(rank), int(first_slot), int(parity_offset_records),
                                                       int(epoch) & 0xFFFFFFFF, current_stream())
        check("launch_khq_publish_partials_fp32", rc)

    def publish_bytes(self, src, nbytes, peer_bufs, dst_byte_offset, peer_flags, flag_index, world, epoch):
        rc = self.lib.launch_khq_publish_bytes(ptr(src), int(nbytes), ptr(peer_bufs), int(dst_byte_offset), ptr(peer_flags),
                                               int(flag_index), int(world), int(epoch) & 0xFFFFFFFF, current_stream())
        check("launch_khq_publish_bytes", rc)

    def wait_flag(self, flag, epoch, max_polls=0):
        rc = self.lib.launch_khq_wait_flag(ptr(flag), int(epoch) & 0xFFFFFFFF, int(max_polls), current_stream())
        check("launch_khq_wait_flag", rc)

    def merge_slots_wait_gate(self, partials, flags, n_flags, epoch, n_slots, q_gate, out, H_q, d, max_polls=0):
        rc = self.lib.launch_khq_merge_slots_wait_gate_fp16(ptr(partials), ptr(flags), int(n_flags), int(epoch) & 0xFFFFFFFF,
                                                            int(n_slots), ptr(q_gate), ptr(out), int(H_q), int(d),
                                                            int(max_polls), current_stream())
        check("launch_khq_merge_slots_wait_gate_fp16", rc)

    # -- launch_khq_gqa_prefill_fp16: causal GQA attention of whole prompts -----------------------
    def gqa_prefill(self, q_gate, k, v, out, batch, T, H_q, H_kv, d, scale):
        """q_gate (batch, T, H_q, 2d), k/v (batch, T, H_kv, d), out (batch, T, H_q, d): contiguous, all
        fp16 (launch_khq_gqa_prefill_fp16) or all bf16 (launch_khq_gqa_prefill_bf16)."""
        dtypes = {getattr(t, "dtype", None) for t in (q_gate, k, v, out)}
        name = "launch_khq_gqa_prefill_fp16"
        if len(dtypes) == 1 and str(next(iter(dtypes))) == "torch.bfloat16":
            name = "launch_khq_gqa_prefill_bf16"
        elif len(dtypes) != 1:
            raise TypeError(f"gqa_prefill: mixed tensor types {dtypes}")
        rc = getattr(self.lib, name)(
            ptr(q_gate), ptr(k), ptr(v), ptr(out), int(batch), int(T), int(H_q), int(H_kv), int(d), float(scale),
            int(T) * H_q * 2 * d, int(T) * H_kv * d, int(T) * H_q * d, current_stream())
        check(name, rc)

    # -- launch_khq_prestep_fp16: q/k head RMSNorm + K capture + partial RoPE + ring appends --------
    def prestep(self, q_gate, k, v, q_norm_w, k_norm_w, ring_k_slot, ring_v_slot, ring_u_slot, H_q, H_kv, d,
                rotary_dim, pos, rope_theta, rms_eps, has_norms):
        rc = self.lib.launch_khq_prestep_fp16(
            ptr(q_gate), ptr(k), ptr(v), ptr(q_norm_w), ptr(k_norm_w), ptr(ring_k_slot), ptr(ring_v_slot),
            ptr(ring_u_slot), int(H_q), int(H_kv), int(d), int(rotary_dim), int(pos), float(rope_theta),
            float(rms_eps), 1 if has_norms else 0, current_stream())
        check("launch_khq_prestep_fp16", rc)

    # -- ring appends (khq_ring_dual_sm75_gpu / copy_vec_sm75_gpu,
    #    src/kernels/elementwise_sm75.mojo:277-312): device-to-device copies ------------------
    # -- launch_khq_cal_kstatic_fp32: K-static fit (op 2 of the reference's launch_cal_op) -------------
    def cal_kstatic(self, rot, rows, cents, out_ts, sigma_out=None):
        rc = self.lib.launch_khq_cal_kstatic_fp32(ptr(rot), int(rows), ptr(cents), ptr(out_ts), ptr(sigma_out), current_stream())
        check("launch_khq_cal_kstatic_fp32", rc)

    def ring_write(self, dst_row, src):
        dst_row.copy_(src.reshape(dst_row.shape), non_blocking=True)

    def synchronize(self):
        import torch

        torch.cuda.current_stream().synchronize()
