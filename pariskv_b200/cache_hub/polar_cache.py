"""ParisKV cache on B200: zone layout, key coding at append, retrieval and sparse decode attention.

Mirror of the reference class ``cache_hub/polar_cache.py:101`` (constructor arguments, the methods
``prefill_update_kv_cache / decode_update_kv_cache / compute / sync`` and the attribute ``context``), so a
model runtime written for the reference decodes through it unchanged.  The body is a different design:

* Per layer there is a small GPU *window* ``[sink | local | update buffer]`` and a *zone store* that
  holds every older token: pinned host memory read through UVA when ``enable_offload`` is set, device
  memory otherwise.  Both modes run the same kernels.
* Zone metadata (sign codes, 4-bit codes, rerank weights) is stored key-major and indexed by the
  zone-relative position, so record 0 is 16-byte aligned and a rerank candidate is two contiguous records.
  ``codebook_gpu / key_block_weight_gpu / key_4bit_packed_gpu`` expose them in the reference's logical
  shapes through permuted views.
* One decode step of one layer is four launches: ``ops.append_encode`` (row append, key coding, flush),
  ``ops.retrieve_ex`` (two launches) and ``ops.sparse_attention``.  No host synchronisation, no concatenation.
* Every position lives in device words (``_layer_state``: rows in the window, searchable keys per sample), read
  by the kernels themselves; the host keeps a mirror for its own decisions.  Launch arguments therefore never
  change: ONE captured CUDA graph serves the whole generation, flushes included.
* A key is coded once, when it is appended (the reference codes a whole update buffer at flush time, for all
  layers at once, and then blocks on its copy stream: cache_hub/polar_cache.py:743-821); its records wait in
  window-aligned staging arrays and are PUBLISHED - copied to the zone, counted in the cluster histogram, K/V row
  sent to the store - when the update buffer fills, so retrieval sees exactly what the reference's lazy index sees.
* Every layer keeps its own counters (the reference derives the slot of every layer from layer 0's counter,
  which makes layers >= 1 lag by one slot).
* Samples of a batch may have different lengths (``valid_start`` per sample, also in lockstep prefill; the
  reference asserts equal lengths, cache_hub/polar_cache.py:396-403): the kernels take the zone length of every
  sample from the device words.
"""
import ctypes
import json
import math
import os

import torch

from .. import _lib, hostmem, ops
from .cache import KV_Cache

USE_RABITQ_RERANK = True
TIER_RATIOS = (0.05, 0.15, 0.30, 0.50, 0.75, 1.0)  # reference: cache_hub/polar_cache.py:1221
ZONE_BOUNDS = (5000, 10000, 30000)                 # zone lengths at which the ratios change (:1113-1124)


def srht_signs(device, seed=42):
    """The SRHT diagonal drawn exactly as the reference draws it (cache_hub/polar_cache.py:56-68):
    seed 42 on the device generator, RNG state restored afterwards."""
    cpu_state = torch.get_rng_state()
    cuda_state = torch.cuda.get_rng_state(device)
    torch.manual_seed(seed)
    signs = torch.randint(0, 2, (128,), device=device, dtype=torch.bfloat16) * 2 - 1
    torch.set_rng_state(cpu_state)
    torch.cuda.set_rng_state(cuda_state, device)
    return signs.contiguous()


class polar_cache(KV_Cache):

    def __init__(self, valid_start, layer_num: int, batch_size: int, max_length: int, num_key_value_heads: int,
                 num_heads: int, head_dim: int, dtype: torch.dtype, layer_mapping: dict, max_new_length: int,
                 sink_size: int, local_size: int, core: int = 0, nprobe: int = 0, cache_unit_size: int = 0,
                 cache_cluster_num: int = 0, num_gpus: int = 1, model_size: int = 0,
                 codebook_path: str = "./turboquant/codebooks/codebook_d128_m8_Kr1_Kw256_rabitq_sign.json",
                 final_topk: int = 100, dynamic_update_interval: int = 512, full_attention_threshold: int = 2000,
                 enable_offload: bool = True, srht_sign_vector=None, per_query_head_retrieval: bool = False) -> None:
        super().__init__(layer_num, batch_size, max_length, num_key_value_heads, num_heads, head_dim, dtype,
                         layer_mapping, num_gpus, model_size)
        if head_dim != 128:
            raise ValueError("the CUDA kernels are built for head_dim 128")
        if dtype != torch.bfloat16:
            raise ValueError("the CUDA kernels are built for bfloat16 K/V")
        self.valid_start = valid_start
        self.sink_size = sink_size
        self.local_size = local_size
        self.steady_size = sink_size + local_size
        self.dynamic_update_interval = dynamic_update_interval if dynamic_update_interval is not None else local_size
        self.group_size = num_heads // num_key_value_heads
        self.max_new_length = max_new_length
        self.input_length = max_length - max_new_length
        self.FULL_ATTENTION_THRESHOLD = full_attention_threshold
        self.final_topk = final_topk
        self.enable_offload = enable_offload
        # Option beyond the reference, which ranks keys by the MEAN of the query heads that share a KV head
        # (cache_hub/polar_cache.py:1026-1031): every query head retrieves its own top-k from its KV head's keys.
        self.per_query_head_retrieval = bool(per_query_head_retrieval)
        self.polar_m, self.polar_K_r, self.polar_K_omega = 8, 1, 256
        if codebook_path and os.path.exists(codebook_path):
            with open(codebook_path) as f:
                cfg = json.load(f)["config"]
            if (cfg["d"], cfg["m"], cfg["K_r"], cfg["K_omega"]) != (128, 8, 1, 256):
                raise ValueError(f"unsupported codebook parameters {cfg}: the kernels implement the sign codebook "
                                 "d=128, m=8, K_r=1, K_omega=256")
        self.polar_B = head_dim // self.polar_m
        self.device = torch.device(list(layer_mapping.values())[0] if layer_mapping else "cuda:0")
        dev = self.device
        self.srht_diagonal_signs = (srht_sign_vector.to(dev, torch.bfloat16).contiguous()
                                    if srht_sign_vector is not None else srht_signs(dev))
        # bf16 roundings of the reference's literals (cache_hub/polar_cache.py:188-193); the thresholds are
        # compiled into the encode kernel, the centers are an operand of the rerank
        self._mag_thresholds = torch.tensor([0.0843, 0.1698, 0.2578, 0.3499, 0.4487, 0.5585, 0.6901],
                                            device=dev, dtype=torch.bfloat16)
        self._mag_centers = torch.tensor([0.0420, 0.1266, 0.2130, 0.3025, 0.3973, 0.5001, 0.6169, 0.7633],
                                         device=dev, dtype=torch.bfloat16)
        I = self.dynamic_update_interval
        self.window_capacity = self.steady_size + I
        self.unified_kv_capacity = self.input_length + self.max_new_length
        # zone capacity: everything that can ever leave the window, rounded up to whole flushes
        zone_cap = max(0, self.unified_kv_capacity - self.steady_size)
        self.zone_capacity = (zone_cap + I - 1) // I * I + I
        bs, H, cap_w = batch_size, self.kv_head, self.window_capacity
        self.unified_keys_gpu = [torch.zeros(bs, H, cap_w, 128, dtype=dtype, device=dev) for _ in range(layer_num)]
        self.unified_values_gpu = [torch.zeros(bs, H, cap_w, 128, dtype=dtype, device=dev) for _ in range(layer_num)]
        # staging records of the window rows (key-major, like the zone records): a key is coded when it is appended and
        # its records are published to the zone when the update buffer is flushed
        self._win_codes = [torch.zeros(bs, H, cap_w, 16, dtype=torch.uint8, device=dev) for _ in range(layer_num)]
        self._win_weight = [torch.zeros(bs, H, cap_w, 16, dtype=torch.bfloat16, device=dev) for _ in range(layer_num)]
        self._win_4bit = [torch.zeros(bs, H, cap_w, 16, 4, dtype=torch.uint8, device=dev) for _ in range(layer_num)]
        self._win_vnorm = [torch.zeros(bs, H, cap_w, dtype=torch.float32, device=dev) for _ in range(layer_num)]
        # device-side positions per layer: [rows in the window, arrival counter, flushes, error flag, keys of sample 0..]
        self._layer_state = [torch.zeros(4 + bs, dtype=torch.int32, device=dev) for _ in range(layer_num)]
        # zone store: the K and V row of a key sit next to each other ([bs,H,cap,2,128]), so a selected key costs one
        # address translation of host memory instead of two; with zones of several GB per layer the row fetch of the
        # attention kernel ran 30 % faster on B200 this way.  unified_keys_cpu / unified_values_cpu are the two
        # strided halves, shaped as the reference's separate tensors.
        if enable_offload:   # page-locked without the pinned allocator's power-of-two rounding
            self._store_kv = [hostmem.pinned_empty(bs, H, self.zone_capacity, 2, 128, dtype=dtype)
                              for _ in range(layer_num)]
            hostmem.release_on_collect(self, list(self._store_kv))
        else:
            self._store_kv = [torch.zeros(bs, H, self.zone_capacity, 2, 128, dtype=dtype, device=dev)
                              for _ in range(layer_num)]
        self._store_k = [t[:, :, :, 0] for t in self._store_kv]
        self._store_v = [t[:, :, :, 1] for t in self._store_kv]
        self.unified_keys_cpu = self._store_k if enable_offload else None
        self.unified_values_cpu = self._store_v if enable_offload else None
        # bulk offload (prefill): device -> pinned host copies run on their own stream so that the compute stream is
        # free for the next layer's prefill; one event per layer, waited for (on the stream, not the host) by the
        # first consumer of that layer's store (cache_hub/polar_cache.py:202-210, :617-639)
        self._copy_stream = torch.cuda.Stream(device=dev) if enable_offload else None
        self._offload_event = [None] * layer_num
        self.BULK_OFFLOAD_ROWS = 4096
        self.codebook_gpu, self.key_block_weight_gpu, self.key_4bit_packed_gpu = [], [], []
        for _ in range(layer_num):
            cb, w, pk = ops.alloc_key_metadata(bs, H, self.zone_capacity, dev)
            self.codebook_gpu.append(cb)
            self.key_block_weight_gpu.append(w)
            self.key_4bit_packed_gpu.append(pk)
        self.cluster_key_counts_gpu = [torch.zeros(bs, H, self.polar_B, 256, dtype=torch.int32, device=dev)
                                       for _ in range(layer_num)]
        # host mirror of the device-side positions
        self.zone_len = [[0] * bs for _ in range(layer_num)]   # searchable keys per layer and sample
        self.cpu_valid_end = [0] * layer_num        # the longest zone of the layer (the zone length when samples agree)
        self.current_seq_len = [0] * layer_num      # tokens seen per layer (longest sample)
        self._window_len = [0] * layer_num          # valid rows of the window per layer
        self._sample_window = [[0] * bs for _ in range(layer_num)]   # the same, per sample, while prefill is under way
        self._all_rows = None
        self.device_positions = True                # positions are always read on the device (kept for callers that ask)
        self.context = 0
        self.last_topk_indices = None               # [bs,H,K] of the most recent compute (for inspection)
        self.last_n_sel = None                      # int32 [bs,H]: valid entries of last_topk_indices
        # Scratch of the retrieval chain and of the attention kernel, sized once for the zone's capacity: the
        # addresses never change, so decode steps captured in CUDA graphs stay valid however the zone grows.
        self._zone_schedule = _lib.zone_schedule(ZONE_BOUNDS, [r[0] for r in self._ratio_rows()],
                                                 [r[1] for r in self._ratio_rows()], TIER_RATIOS)
        c_max = int(_lib.load().pk_zone_max_candidates(ctypes.byref(self._zone_schedule), max(self.zone_capacity, 1)))
        self._c_max = max(c_max, 1)
        rows = (bs * H, self.group_size) if self.per_query_head_retrieval else (bs, H)
        self._retrieve_scratch = ops.Scratch(dev, ops.retrieve_scratch_bytes(rows[0], rows[1], max(self.zone_capacity, 1), self._c_max))
        self._attn_rows_max = self.window_capacity + max(self.final_topk, self._max_selected_rows())
        self.queries_precede_append = False   # see compute(): set by callers that make q and k in one kernel
        self._appended_layer = None
        self._attn_scratch = ops.Scratch(dev, ops.attention_scratch_bytes(bs, num_heads, self._attn_rows_max))

    def _max_selected_rows(self):
        """Most zone rows one attention call can be given besides the window: the full-attention regime attends every
        zone row while the sequence is shorter than the threshold."""
        return max(self.FULL_ATTENTION_THRESHOLD, self.steady_size + 2 * self.final_topk)

    def _zone_vnorm(self, layer):
        """fp32 ||v|| of the zone rows, kept by the variants that rank candidates by it (None here)."""
        return None

    def _attend(self, queries, wk, wv, n_win, *args, **kw):
        """ops.sparse_attention on the cache's own scratch (the shared, growable one for an oversized eager call)."""
        sel = args[2] if len(args) > 2 else kw.get("selected")
        rows = n_win + (sel.shape[2] if sel is not None else 0)
        scratch = self._attn_scratch if rows <= self._attn_rows_max else None
        return ops.sparse_attention(queries, wk, wv, n_win, *args, scratch=scratch, **kw)

    def check_status(self):
        """Raise if a kernel reported a problem through its status word: an attention block whose row copies never
        landed, an append into a full window, a flush into a full zone (a host synchronisation: call it between
        decode loops, not inside one)."""
        ops.check_attention_status(self._attn_scratch, self.batch_size, self.num_heads)
        flags = torch.stack([s[3] for s in self._layer_state]).cpu()
        if int(flags.abs().sum()) != 0:
            raise RuntimeError("append: a layer's window was overrun or its zone / store had no room for a flush "
                               f"(layers {[i for i, f in enumerate(flags.tolist()) if f]})")

    # ------------------------------------------------------------------------------------------------
    # prefill
    # ------------------------------------------------------------------------------------------------
    def prefill_update_kv_cache(self, query_states, key_states, value_states, layer_idx, batch_idx):
        """key_states / value_states: [bsz, seq_len, kv_heads, 128].  bsz == 1 fills sample `batch_idx`;
        bsz == batch_size fills all samples at once, each from its own valid_start (left padding; the reference
        requires equal valid_start in this form, cache_hub/polar_cache.py:396-403).  Returns the K/V to attend in
        the prefill itself, as the reference does (:379-387)."""
        bsz, seq_len = key_states.shape[:2]
        assert seq_len <= self.input_length, "prompt longer than the cache was sized for"
        if bsz == 1:
            vs = self._valid_start(batch_idx)
            self._prefill_sample(key_states[0], value_states[0], layer_idx, batch_idx, vs)
            last = batch_idx + 1 == self.batch_size
        else:
            vs = min(self._valid_start(b) for b in range(bsz))
            if batch_idx != 0:
                return key_states[:, vs:], value_states[:, vs:]
            assert bsz == self.batch_size, "lockstep prefill needs the whole batch"
            for b in range(bsz):
                self._prefill_sample(key_states[b], value_states[b], layer_idx, b, self._valid_start(b))
            last = True
        if last:
            if len(set(self._sample_window[layer_idx])) > 1:
                raise ValueError("the samples of a batch must fill the same number of window rows: prompts of a batch "
                                 f"must all be at least sink + local = {self.steady_size} tokens long, or equally long")
            longest = max(seq_len - self._valid_start(b) for b in range(self.batch_size))
            self.current_seq_len[layer_idx] = longest
            self.cpu_valid_end[layer_idx] = max(self.zone_len[layer_idx])
            st = [self._window_len[layer_idx], 0, 0, 0] + list(self.zone_len[layer_idx])
            self._layer_state[layer_idx].copy_(torch.tensor(st, dtype=torch.int32), non_blocking=False)
            if layer_idx == self.layer_num - 1:
                self.context += longest
        return key_states[:, vs:], value_states[:, vs:]

    def _valid_start(self, b):
        vs = self.valid_start     # a number, or one per sample (list, tensor, numpy array: the reference passes the latter)
        if getattr(vs, "ndim", None) == 0 or not hasattr(vs, "__len__"):
            return int(vs)
        return int(vs[b])

    def _prefill_sample(self, k, v, layer, b, vs):
        """k, v: [seq_len, H, 128] of one sample; tokens before `vs` are padding."""
        k = k[vs:].to(self.dtype)
        v = v[vs:].to(self.dtype)
        P = k.shape[0]
        sink, local = self.sink_size, self.local_size
        wk, wv = self.unified_keys_gpu[layer], self.unified_values_gpu[layer]
        N = max(0, P - self.steady_size)
        if N == 0:  # short prompt: everything stays in the window
            n = min(P, self.window_capacity)
            wk[b, :, :n] = k[:n].transpose(0, 1)
            wv[b, :, :n] = v[:n].transpose(0, 1)
        else:
            n = self.steady_size
            wk[b, :, :sink] = k[:sink].transpose(0, 1)
            wv[b, :, :sink] = v[:sink].transpose(0, 1)
            wk[b, :, sink:sink + local] = k[P - local:].transpose(0, 1)
            wv[b, :, sink:sink + local] = v[P - local:].transpose(0, 1)
            zk = k[sink:sink + N].transpose(0, 1)   # [H, N, 128] strided view, rows 16-byte aligned
            zv = v[sink:sink + N].transpose(0, 1)
            self._append_zone(layer, b, zk, zv, 0, N, reset_counts=True)
        if N == 0:
            self.cluster_key_counts_gpu[layer][b].zero_()
        self._stage_window_rows(layer, b, n)
        self._window_len[layer] = n
        self._sample_window[layer][b] = n
        self.zone_len[layer][b] = N

    def _stage_window_rows(self, layer, b, n):
        """Code the first n window rows of sample b into the staging arrays (the rows behind the sink will be flushed
        later; their records must be ready) and record their value norms."""
        if n <= 0:
            return
        wk, wv = self.unified_keys_gpu[layer], self.unified_values_gpu[layer]
        view = lambda t: t[b:b + 1, :, :n].permute(0, 1, 3, 2)              # key-major storage, reference-shaped view
        ops.encode_keys(wk[b:b + 1, :, :n], self.srht_diagonal_signs, view(self._win_codes[layer]),
                        view(self._win_weight[layer]), self._win_4bit[layer][b:b + 1, :, :n].permute(0, 1, 3, 2, 4))
        self._win_vnorm[layer][b, :, :n] = torch.linalg.vector_norm(wv[b, :, :n].float(), dim=-1)

    def _append_zone(self, layer, b, zk, zv, start, n, reset_counts=False):
        """Code n keys ([H, n, 128]) of sample b into zone records [start, start+n) and copy K/V to the store."""
        sl = slice(start, start + n)
        counts = self.cluster_key_counts_gpu[layer][b:b + 1]
        if reset_counts:
            counts.zero_()
        ops.encode_keys(zk.unsqueeze(0), self.srht_diagonal_signs,
                        self.codebook_gpu[layer][b:b + 1, :, :, sl], self.key_block_weight_gpu[layer][b:b + 1, :, :, sl],
                        self.key_4bit_packed_gpu[layer][b:b + 1, :, :, sl, :], cluster_counts=counts)
        skv = self._store_kv[layer]
        kv = torch.stack((zk, zv), dim=2)  # [H, n, 2, 128] on the device: K and V rows interleaved as the store holds them
        if self._copy_stream is not None and n >= self.BULK_OFFLOAD_ROWS:
            cur = torch.cuda.current_stream(kv.device)
            self._wait_offload(layer)                 # an earlier bulk copy of this layer must stay ordered
            self._copy_stream.wait_stream(cur)
            with torch.cuda.stream(self._copy_stream):
                for h in range(self.kv_head):
                    skv[b, h, sl].copy_(kv[h], non_blocking=True)
                ev = torch.cuda.Event()
                ev.record(self._copy_stream)
            kv.record_stream(self._copy_stream)       # keep the staging tensor alive until the copies have run
            self._offload_event[layer] = ev
            return
        self._wait_offload(layer)
        for h in range(self.kv_head):  # contiguous per-head blocks: one async copy each, on the current stream
            skv[b, h, sl].copy_(kv[h], non_blocking=True)

    def _wait_offload(self, layer):
        """Order the current stream after the layer's pending bulk offload, if any (no host block)."""
        ev = self._offload_event[layer]
        if ev is not None:
            torch.cuda.current_stream().wait_event(ev)
            self._offload_event[layer] = None

    # ------------------------------------------------------------------------------------------------
    # decode
    # ------------------------------------------------------------------------------------------------
    def decode_update_kv_cache(self, key_states, value_states, layer_idx):
        """Append the step's K/V row ([bs, 1, H, 128]): one launch that writes the row, codes the key and, when the
        row fills the window, flushes the update buffer into the zone (reference: decode_update_kv_cache +
        _update_polar_index, cache_hub/polar_cache.py:827-881, :743-821)."""
        l = layer_idx
        if self._window_len[l] + 1 == self.window_capacity and max(self.zone_len[l]) + self.dynamic_update_interval > self.zone_capacity:
            raise RuntimeError("zone store is full: construct the cache with a larger max_length / max_new_length")
        self._wait_offload(l)      # the flush writes store rows: stay ordered behind a pending bulk offload
        ops.append_encode(key_states, value_states, self.srht_diagonal_signs, self.unified_keys_gpu[l],
                          self.unified_values_gpu[l], self._win_codes[l], self._win_weight[l], self._win_4bit[l],
                          self._win_vnorm[l], self.codebook_gpu[l], self.key_block_weight_gpu[l],
                          self.key_4bit_packed_gpu[l], self._zone_vnorm(l), self.cluster_key_counts_gpu[l],
                          self._store_kv[l], self._layer_state[l], self.sink_size, self.dynamic_update_interval)
        self._mirror_append(l)
        self._appended_layer = l
        if l == 0:
            self.context += 1
        return None, None

    def _mirror_append(self, l):
        """The host-side copy of what the append kernel does to the layer's positions."""
        self._window_len[l] += 1
        self.current_seq_len[l] += 1
        if self._window_len[l] == self.window_capacity:
            I = self.dynamic_update_interval
            self.zone_len[l] = [n + I for n in self.zone_len[l]]
            self.cpu_valid_end[l] += I
            self._window_len[l] = self.window_capacity - I

    # ------------------------------------------------------------------------------------------------
    # attention
    # ------------------------------------------------------------------------------------------------
    def _ratio_rows(self):
        """(candidate_ratio, collision_ratio) for zones shorter than ZONE_BOUNDS[i], and for the rest:
        cache_hub/polar_cache.py:1113-1124."""
        return [(0.5, 0.5), (0.25, 0.3), (0.2, 0.25), (0.1, 0.2)]

    def _get_adaptive_ratios(self, retrieval_len):
        rows = self._ratio_rows()
        for bound, row in zip(ZONE_BOUNDS, rows):
            if retrieval_len < bound:
                return row
        return rows[-1]

    def retrieval_plan(self, N):
        """(tier thresholds, candidate count C, final K) for a zone of N keys
        (cache_hub/polar_cache.py:1221-1222, :1239-1240, :1300).  The kernels compute the same numbers from the
        device-side zone length."""
        cand_ratio, coll_ratio = self._get_adaptive_ratios(N)
        tiers = [int(math.ceil(N * coll_ratio * r)) for r in TIER_RATIOS]
        C = max(1, int(math.ceil(N * cand_ratio)))
        return tiers, C, min(self.final_topk, C)

    def _full_regime(self, layer_idx):
        """True while the sequence is short enough to attend every zone row (cache_hub/polar_cache.py:1033-1045)."""
        total = self.current_seq_len[layer_idx]
        return total < max(self.FULL_ATTENTION_THRESHOLD, self.steady_size + 2 * self.final_topk) or self.cpu_valid_end[layer_idx] <= 0

    def graph_key(self):
        """What a captured decode step depends on besides the device words: which of the two attention regimes the
        host picked.  Callers that replay CUDA graphs keep one graph per key."""
        return "full" if self._full_regime(0) else "retrieve"

    def compute(self, queries, layer_idx):
        """Decode attention of one token: queries [bs, 1, num_heads, 128] -> [bs, 1, num_heads, 128]."""
        queries = queries.contiguous()
        self._wait_offload(layer_idx)
        l = layer_idx
        st = self._layer_state[l]
        wk, wv = self.unified_keys_gpu[l], self.unified_values_gpu[l]
        sk, sv = self._store_k[l], self._store_v[l]
        if self._full_regime(l):  # attend everything (eager only: the row count is a host number)
            N, n_win = self.cpu_valid_end[l], self._window_len[l]
            if min(self.zone_len[l]) != N:
                raise RuntimeError("full attention over short sequences needs samples of equal length")
            if N <= 0:
                return self._attend(queries, wk, wv, n_win)
            if self._all_rows is None or self._all_rows.shape[-1] < N:
                self._all_rows = torch.arange(self.zone_capacity, device=self.device).expand(
                    self.batch_size, self.kv_head, -1).contiguous()
            sel = self._all_rows[:, :, :N].contiguous() if N != self._all_rows.shape[-1] else self._all_rows
            return self._attend(queries, wk, wv, n_win, sk, sv, sel)
        if self.per_query_head_retrieval:
            return self._compute_per_query_head(queries, l)
        # A caller whose queries are made BEFORE it calls decode_update_kv_cache (one kernel makes q and k) says so with
        # queries_precede_append: the append launch of this layer then sits between that kernel and this call, and the
        # collision kernel may prepare the query before it waits for the append (matters with dependent launch only).
        settled = self.queries_precede_append and self._appended_layer == l
        self._appended_layer = None
        final, n_sel, _ = ops.retrieve_ex(queries, self.srht_diagonal_signs, self._mag_centers, self.codebook_gpu[l],
                                          self.key_block_weight_gpu[l], self.key_4bit_packed_gpu[l],
                                          self.cluster_key_counts_gpu[l], self._c_max, self.final_topk,
                                          kv_len=st[4:4 + self.batch_size], schedule=self._zone_schedule,
                                          scratch=self._retrieve_scratch, queries_settled=settled)
        self._remember_selection(final, n_sel, l)
        # window rows and zone rows per head are read on the device
        return self._attend(queries, wk, wv, self.window_capacity, sk, sv, final, n_sel=n_sel,
                            n_window_dev=st[0:1], n_window_add=0)

    def _remember_selection(self, final, n_sel, l):
        """last_topk_indices as the reference exposes it: [bs,H,K] with K = min(final_topk, candidates) when the
        samples agree on the zone length; with per-sample lengths the full rows plus last_n_sel."""
        self.last_n_sel = n_sel
        if min(self.zone_len[l]) == max(self.zone_len[l]):
            final = final[:, :, :self.retrieval_plan(self.zone_len[l][0])[2]]
        self.last_topk_indices = final

    def _compute_per_query_head(self, queries, l):
        """Retrieval and attention with one selection per QUERY head.  Nothing is copied: every (batch, KV head)
        becomes a batch entry whose G "heads" all point at that KV head's keys (stride 0 over the group), and the
        same kernels run with a group size of one."""
        bs, H, G = self.batch_size, self.kv_head, self.group_size
        st = self._layer_state[l]

        def per_group(t):   # [bs,H,...] -> [bs*H, G, ...], the group dimension with stride 0
            return t.view(bs * H, 1, *t.shape[2:]).expand(bs * H, G, *t.shape[2:])

        q = queries.view(bs, H, G, 128).reshape(bs * H, 1, G, 128)
        counts = per_group(self.cluster_key_counts_gpu[l]).contiguous()
        kv_len = st[4:4 + bs].repeat_interleave(H)          # one entry per (batch, KV head)
        final, n_sel, _ = ops.retrieve_ex(q, self.srht_diagonal_signs, self._mag_centers, per_group(self.codebook_gpu[l]),
                                          per_group(self.key_block_weight_gpu[l]), per_group(self.key_4bit_packed_gpu[l]),
                                          counts, self._c_max, self.final_topk, kv_len=kv_len,
                                          schedule=self._zone_schedule, scratch=self._retrieve_scratch)
        self._remember_selection(final.view(bs, H * G, -1), n_sel.view(bs, H * G), l)   # one row per query head
        wk, wv = per_group(self.unified_keys_gpu[l]), per_group(self.unified_values_gpu[l])
        sk, sv = per_group(self._store_k[l]), per_group(self._store_v[l])
        out = self._attend(q, wk, wv, self.window_capacity, sk, sv, final, n_sel=n_sel, n_window_dev=st[0:1],
                           n_window_add=0)
        return out.view(bs, 1, H * G, 128)

    # ------------------------------------------------------------------------------------------------
    # support for replaying a captured decode step
    # ------------------------------------------------------------------------------------------------
    def next_step_flushes(self) -> bool:
        """Never: the flush is part of the append launch and reads its positions on the device, so the step that
        flushes is captured and replayed like any other."""
        return False

    def sync_device_state(self):
        """Nothing to do: the device words are advanced by the append kernel itself."""

    def advance_device_step(self):
        """Nothing to do (see sync_device_state)."""

    def host_state(self):
        return ([list(z) for z in self.zone_len], list(self._window_len), list(self.current_seq_len), self.context,
                list(self.cpu_valid_end))

    def set_host_state(self, st):
        self.zone_len, self._window_len = [list(z) for z in st[0]], list(st[1])
        self.current_seq_len, self.context, self.cpu_valid_end = list(st[2]), st[3], list(st[4])

    def host_state_after_flushes(self, j):
        """None: no graph has to be captured ahead of time, one graph covers every zone length."""
        return None

    def note_replayed_step(self):
        """Host-side bookkeeping of one decode step that ran as a graph replay."""
        for l in range(self.layer_num):
            self._mirror_append(l)
        self.context += 1

    def sync(self, layer_idx, batch_idx):
        """Order the current stream after the layer's bulk offload (cache_hub/polar_cache.py:617-639).  The
        reference blocks the host here; a stream-side wait is enough because every consumer is a kernel."""
        self._wait_offload(layer_idx)
        return None
