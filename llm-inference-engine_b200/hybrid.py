"""The layer-list decoder (b200_hybrid_*, csrc/hybrid.cu) behind a small class: a model is a list of layer descriptions -- a token
mixer of some kind plus an optional feed-forward of some kind, each with its sizes, constants and device tensors -- and one `forward`
runs a ragged mixed batch (portions of prompts beside single decoded tokens) against the paged key/value pool and the state slots."""
import ctypes as C
import importlib

import numpy as np


def _mod():
    return importlib.import_module(__package__ or "llm-inference-engine_b200")


class HybridDecoder:
    """layers: list of dicts with the integer / float fields of b200_hybrid_layer_t and device tensors under the weight names.
    The tensors are kept alive by this object."""

    def __init__(self, width, vocab, eps, layers, embedding, final_norm, lm_head, dtype, device, max_tokens, max_seqs, max_pages_per_seq,
                 embed_scale=1.0, logit_softcap=0.0, final_norm_kind=0, loop=None, logit_scale=1.0, streams=0):
        """loop: None, or dict(start, stop, times[, w_entry [width, 2*width] of the engine dtype, step fp32 [times, width]]): the layers
        start .. stop-1 run `times` times with the same weights; shared-norm layers open every pass with the entry step
        x <- w_entry [x ; x0] + step[pass].  streams: residual streams of pre-norm layers (0: one)."""
        import torch

        m = _mod()
        self.device = torch.device(device)
        self.torch_dtype = dtype
        code = {torch.float32: m.F32, torch.float16: m.F16, torch.bfloat16: m.BF16}[dtype]
        self.cfg = m.HybridConfig(int(width), int(vocab), len(layers), code, float(eps), int(max_tokens), int(max_seqs), int(max_pages_per_seq),
                                  float(embed_scale), float(logit_softcap), int(final_norm_kind),
                                  int(loop["start"]) if loop else 0, int(loop["stop"]) if loop else 0, int(loop["times"]) if loop else 0,
                                  float(logit_scale), int(streams))
        self.handle = m.lib().b200_hybrid_create(C.byref(self.cfg))
        if not self.handle:
            raise m.B200Error(m.lib().b200_last_error_string().decode())
        self._keep = [layers, embedding, final_norm, lm_head, loop]
        self.layers = layers
        ints = ("mixer", "heads", "kv_heads", "dim", "vdim", "chunk", "decay_rank", "mlp", "experts", "top", "expert_ff", "shared_ff", "act",
                "norm", "window", "kv_rank", "rot_dim", "rot_dims", "route", "identity", "gated", "attn_weight", "out_gate", "conv", "gate_rank",
                "rot_half", "v_norm", "gate_act", "norm_groups")
        tensors = ("w_in", "w_out", "q_norm", "k_norm", "sink", "w_decay", "decay_bias", "out_norm", "norm1", "norm2", "w_router", "w_up",
                   "w_down", "w_shared_up", "w_shared_down", "kv_norm", "w_uk_t", "w_uv", "pre1", "post1", "pre2", "post2", "ls1", "ls2",
                   "route_bias", "b_up", "b_down", "head_bias", "dist_r1", "dist_r2", "b_in", "b_out", "conv_w", "a_log", "w_gate2", "conv_b", "skip",
                   "head_decay", "hc1", "hc2", "branch_norm")
        f32_vectors = {"q_norm", "k_norm", "sink", "decay_bias", "out_norm", "norm1", "norm2", "kv_norm", "pre1", "post1", "pre2", "post2",
                       "ls1", "ls2", "route_bias", "b_up", "b_down", "head_bias", "dist_r1", "dist_r2", "b_in", "b_out", "conv_w", "a_log", "conv_b", "skip",
                       "head_decay", "hc1", "hc2", "branch_norm"}

        def fill(spec, where):
            lw = m.HybridLayer()
            for k in ints:
                setattr(lw, k, int(spec.get(k, 0)))
            lw.scale, lw.tau = float(spec.get("scale", 1.0)), float(spec.get("tau", 1.0))
            lw.rot_base, lw.kv_from = float(spec.get("rot_base", 0.0)), int(spec.get("kv_from", -1))
            lw.gate_cap, lw.mix_scale, lw.side_scale = float(spec.get("gate_cap", 0.0)), float(spec.get("mix_scale", 1.0)), float(spec.get("side_scale", 1.0))
            for k in ("rot_factor", "rot_low", "rot_high", "rot_original", "softcap"):
                setattr(lw, k, float(spec.get(k, 0.0)))
            for k in tensors:
                t = spec.get(k)
                if t is not None:
                    want = torch.float32 if k in f32_vectors else dtype
                    assert t.is_cuda and t.is_contiguous() and t.dtype == want, f"{where}: tensor {k} must be a contiguous {want} CUDA tensor"
                    setattr(lw, k, t.data_ptr())
            return lw

        for i, spec in enumerate(layers):
            lw = fill(spec, f"layer {i}")
            if spec.get("side") is not None:  # a second mixer beside the first (the engine copies it)
                side = fill(spec["side"], f"layer {i} (second mixer)")
                lw.side = C.addressof(side)
            m.check(m.lib().b200_hybrid_set_layer(self.handle, i, C.byref(lw)))
        if loop and loop.get("w_entry") is not None:
            assert loop["w_entry"].dtype == dtype and loop["w_entry"].is_contiguous() and loop["step"].dtype == torch.float32 and loop["step"].is_contiguous()
            m.check(m.lib().b200_hybrid_set_loop(self.handle, m.ptr(loop["w_entry"]), m.ptr(loop["step"])))
        self.num_runs = m.lib().b200_hybrid_num_runs(self.handle)
        assert embedding.dtype == dtype and lm_head.dtype == dtype and final_norm.dtype == torch.float32
        m.check(m.lib().b200_hybrid_set_io(self.handle, m.ptr(embedding), m.ptr(final_norm), m.ptr(lm_head)))
        nbytes = m.lib().b200_hybrid_scratch_bytes(self.handle)
        self._scratch = torch.empty(nbytes + 256, dtype=torch.uint8, device=self.device)
        base = (self._scratch.data_ptr() + 255) // 256 * 256
        m.check(m.lib().b200_hybrid_set_scratch(self.handle, C.c_void_p(base), nbytes))
        self.kv_pool = self.state_pool = None
        m.ensure_workspace()

    def __del__(self):
        if getattr(self, "handle", None):
            try:
                _mod().lib().b200_hybrid_destroy(self.handle)
            except Exception:  # interpreter shutdown: the module table is already gone
                pass
            self.handle = None

    def set_pools(self, num_pages, num_slots, poison=False):
        """Allocates the key/value pool (num_pages pages of KV_PAGE_SIZE positions) and the state pool (num_slots slots)."""
        import torch

        m = _mod()
        kb = m.lib().b200_hybrid_kv_pool_bytes(self.handle, int(num_pages))
        sb = m.lib().b200_hybrid_state_pool_bytes(self.handle, int(num_slots))
        self.kv_pool = torch.zeros(kb + 256, dtype=torch.uint8, device=self.device)
        self.state_pool = torch.zeros(sb + 256, dtype=torch.uint8, device=self.device)
        if poison:  # tests: whatever is read without having been written shows
            self.kv_pool.fill_(0xFF)
            self.state_pool.fill_(0xFF)
        kp = (self.kv_pool.data_ptr() + 255) // 256 * 256
        sp = (self.state_pool.data_ptr() + 255) // 256 * 256
        m.check(m.lib().b200_hybrid_set_pools(self.handle, C.c_void_p(kp), int(num_pages), C.c_void_p(sp), int(num_slots)))
        self.num_pages, self.num_slots = int(num_pages), int(num_slots)

    def forward(self, token_ids, seq_start, seq_pos0, seq_slot, block_table, want_rows, trace=False):
        """Host integer arrays in, device fp32 logits [len(want_rows), vocab] out (and, with trace=True, the residual stream after
        every layer run, [runs, tokens, width])."""
        import torch

        m = _mod()
        a = [np.ascontiguousarray(np.asarray(v, dtype=np.int32)) for v in (token_ids, seq_start, seq_pos0, seq_slot, block_table, want_rows)]
        n_tokens, n_seqs, n_want = int(a[0].size), int(a[2].size), int(a[5].size)
        assert a[4].size == n_seqs * self.cfg.max_pages_per_seq, "block_table must be [n_seqs, max_pages_per_seq]"
        hb = m.HybridBatch(n_tokens, n_seqs, n_want, *[v.ctypes.data_as(C.c_void_p) for v in a])
        logits = torch.empty((n_want, self.cfg.vocab), dtype=torch.float32, device=self.device)
        tr = torch.empty((self.num_runs, n_tokens, self.cfg.width), dtype=torch.float32, device=self.device) if trace else None
        m.check(m.lib().b200_hybrid_forward(self.handle, C.byref(hb), m.ptr(logits) if n_want else None, m.ptr(tr) if trace else None, m.stream()))
        return (logits, tr) if trace else logits
