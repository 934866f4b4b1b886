"""Shared body of the two adaptive-k cache variants: value-norm bookkeeping and the adaptive selection step.

Both variants keep all C rerank candidates, weight them by exp(logit - max) * ||v|| together with the window
rows, and attend the shortest benefit-ordered prefix that reaches a share `threshold` of the total benefit
(reference: cache_hub/polar_cache_atten_value_indices_adaptive_k.py:1510-1589,
cache_hub/polar_cache_adaptivek_varlen.py:1684-1812).  Here the selection is one kernel
(ops.adaptive_topk), the value norms of the candidates are gathered inside it, and the attention kernel takes
per-head row counts, so there is no host synchronisation, no index packing and no staging copy.
"""
import math

import torch

from .. import ops
from .polar_cache import polar_cache as _base_cache


class AdaptiveKCache(_base_cache):
    # (candidate_ratio, collision_ratio) by zone length, adaptive variants
    # (cache_hub/polar_cache_adaptivek_varlen.py:2115-2126)
    def _ratio_rows(self):
        return [(0.5, 0.5), (0.25, 0.3), (0.2, 0.25), (0.05, 0.2)]

    def _max_selected_rows(self):
        return max(super()._max_selected_rows(), 4096)   # the adaptive selection may attend up to 4096 rows per head

    def _init_adaptive(self, threshold, min_k, max_k, per_head):
        self.adaptive_topk_threshold = float(threshold)
        self._min_k, self._max_k, self._per_head = int(min_k), int(max_k), bool(per_head)
        if self._max_k > 4096:
            raise ValueError("adaptive top-k supports at most 4096 rows per head")
        dev, bs, H = self.device, self.batch_size, self.kv_head
        self._attn_scale = 1.0 / math.sqrt(self.head_dim)
        # ||v|| of the window rows and of the zone rows (zone-relative index), fp32.  The window norms are the staging
        # array that the append kernel fills for every cache; the zone norms are published by its flush.
        self._sl_vnorm_cache = self._win_vnorm
        self.value_norm_gpu = [torch.zeros(bs, H, self.zone_capacity, dtype=torch.float32, device=dev)
                               for _ in range(self.layer_num)]
        self.last_adaptive = None   # (adaptive_k, topk_indices, n_sel, sl_logits, cand, cand_scores) of the last compute
        self.fixed_shapes = False   # True: capacity-shaped tensors on eager steps too (what a stream capture uses)
        self._row_ids = torch.arange(self.window_capacity, device=dev, dtype=torch.int32)

    def _zone_vnorm(self, layer):
        return self.value_norm_gpu[layer]

    # ---- value norms of the prompt (decode rows are handled by the append kernel) -------------------------
    def _prefill_sample(self, k, v, layer, b, vs):
        super()._prefill_sample(k, v, layer, b, vs)
        N = self.zone_len[layer][b]
        if N > 0:
            vn = torch.linalg.vector_norm(v[vs:].to(self.dtype).float(), dim=-1).transpose(0, 1)  # [H, P]
            self.value_norm_gpu[layer][b, :, :N] = vn[:, self.sink_size:self.sink_size + N]

    # ---- decode attention ---------------------------------------------------------------------------------
    def compute(self, queries, layer_idx):
        queries = queries.contiguous()
        self._wait_offload(layer_idx)
        N = self.cpu_valid_end[layer_idx]
        n_win = self._window_len[layer_idx]
        total = self.current_seq_len[layer_idx]
        if total < max(self.FULL_ATTENTION_THRESHOLD, self.steady_size + 2 * self.final_topk) or N <= 0:
            return super().compute(queries, layer_idx)
        wk, wv = self.unified_keys_gpu[layer_idx], self.unified_values_gpu[layer_idx]
        # rows of the candidate lists are c_max long; a sample's own count follows from its zone length, read on the
        # device, and the rest of its row carries score -inf (no weight in the adaptive selection)
        st = self._layer_state[layer_idx]
        _, _, ex = ops.retrieve_ex(queries, self.srht_diagonal_signs, self._mag_centers, self.codebook_gpu[layer_idx],
                                   self.key_block_weight_gpu[layer_idx], self.key_4bit_packed_gpu[layer_idx],
                                   self.cluster_key_counts_gpu[layer_idx], self._c_max, 0, kv_len=st[4:4 + self.batch_size],
                                   schedule=self._zone_schedule, want=("cand", "scores_f32", "query_avg"),
                                   scratch=self._retrieve_scratch)
        cand, cand_scores = ex["cand"], ex["scores_f32"]
        C = self.retrieval_plan(N)[1]          # candidates of the longest sample
        # Shapes that follow the host's view of the lengths (the reference's shapes) on eager steps; inside a stream
        # capture, or with fixed_shapes set, every shape is a capacity and the lengths act on the device only: window
        # rows beyond the filled part get logit -inf, candidate rows keep their -inf tail, and a head never attends
        # more rows than it has candidates.  Both forms attend the same rows.
        fixed = self.fixed_shapes or torch.cuda.is_current_stream_capturing()
        equal = min(self.zone_len[layer_idx]) == N
        if fixed:
            n_rows, C = self.window_capacity, cand.shape[2]
        else:
            n_rows = n_win
            if equal:   # equal lengths: the lists as the reference shapes them, [bs,H,C]
                cand, cand_scores = cand[:, :, :C].contiguous(), cand_scores[:, :, :C].contiguous()
        cand_scores = cand_scores.to(torch.bfloat16)   # the reference ranks bf16 scores
        # window logits: a small dense product, left to the library as the reference does
        sl_logits = torch.einsum("bhd,bhkd->bhk", ex["query_avg"], wk[:, :, :n_rows]).to(torch.float32) * self._attn_scale
        if fixed:
            sl_logits = sl_logits.masked_fill(self._row_ids[:n_rows] >= st[0], float("-inf"))
        K_out = min(self._max_k, C)
        min_k = min(self._min_k, K_out)
        adaptive_k, topk = ops.adaptive_topk(sl_logits.contiguous(), cand_scores, self._attn_scale,
                                             self._sl_vnorm_cache[layer_idx][:, :, :n_rows], cand, None,
                                             self.adaptive_topk_threshold, K_out,
                                             value_norm=self.value_norm_gpu[layer_idx], sink_size=0,
                                             min_k=max(1, min_k), max_k=max(1, K_out))
        if fixed or not equal:   # rows longer than a sample's candidate list: its count caps what the head attends
            adaptive_k = torch.minimum(adaptive_k, ex["n_cand"].to(adaptive_k.dtype))
        if self._per_head:
            n_sel = adaptive_k.to(torch.int32)
        else:  # dense variant: every head attends the first max-over-heads rows of its own ranking
            n_sel = adaptive_k.max().to(torch.int32).expand_as(adaptive_k).contiguous()
            if fixed or not equal:
                n_sel = torch.minimum(n_sel, ex["n_cand"])
        self.last_adaptive = (adaptive_k, topk, n_sel, sl_logits, cand, cand_scores)
        self.last_topk_indices = topk
        if fixed:
            return self._attend(queries, wk, wv, self.window_capacity, self._store_k[layer_idx], self._store_v[layer_idx],
                                topk, n_sel=n_sel, n_window_dev=st[0:1], n_window_add=0)
        return self._attend(queries, wk, wv, n_win, self._store_k[layer_idx], self._store_v[layer_idx], topk,
                            n_sel=n_sel)
