"""ParisKV cache on B200: zone layout, key coding at flush, retrieval and sparse decode attention.

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
* One decode step of one layer is: a row append, ``ops.retrieve`` (five launches), ``ops.sparse_attention``
  (two launches).  No host synchronisation, no allocation, no concatenation.
* The window position can be read on the device (``device_positions``): the row append and the attention
  then take the window length from a device word instead of a launch argument, so a whole decode step can
  be captured in a CUDA graph and replayed until the next flush.
* Every layer keeps its own buffer counter (the reference derives the slot of every layer from layer 0's
  counter, which makes layers >= 1 lag by one slot); a layer flushes its own buffer when it fills:
  the oldest ``dynamic_update_interval`` local rows are coded, added to the cluster histogram, copied to the
  zone store on the same stream, and the window slides.
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
                 enable_offload: bool = True, srht_sign_vector=None) -> None:
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
        bs, H = batch_size, self.kv_head
        self.unified_keys_gpu = [torch.zeros(bs, H, self.window_capacity, 128, dtype=dtype, device=dev)
                                 for _ in range(layer_num)]
        self.unified_values_gpu = [torch.zeros(bs, H, self.window_capacity, 128, dtype=dtype, device=dev)
                                   for _ in range(layer_num)]
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
        self.cpu_valid_end = [0] * layer_num        # searchable keys per layer (zone length N)
        self.current_seq_len = [0] * layer_num      # tokens seen per layer
        self._window_len = [0] * layer_num          # valid rows of the window per layer
        self._slide_tmp_k = torch.empty(bs, H, max(local_size, 1), 128, dtype=dtype, device=dev)
        self._slide_tmp_v = torch.empty_like(self._slide_tmp_k)
        self._all_rows = None
        # device copy of the window length at the start of the current step (all layers agree between steps)
        self._dev_state = torch.zeros(2, dtype=torch.int32, device=dev)
        self.device_positions = False
        self.context = 0
        self.last_topk_indices = None               # [bs,H,K] of the most recent compute (for inspection)
        # Scratch of the retrieval chain and of the attention kernel, sized once for the zone's capacity: the
        # addresses never change, so decode steps captured in CUDA graphs stay valid however the zone grows.
        self._zone_schedule = _lib.zone_schedule(ZONE_BOUNDS, [r[0] for r in self._ratio_rows()],
                                                 [r[1] for r in self._ratio_rows()], TIER_RATIOS)
        c_max = int(_lib.load().pk_zone_max_candidates(ctypes.byref(self._zone_schedule), max(self.zone_capacity, 1)))
        self._c_max = max(c_max, 1)
        self._retrieve_scratch = ops.Scratch(dev, ops.retrieve_scratch_bytes(bs, H, max(self.zone_capacity, 1), self._c_max))
        self._attn_rows_max = self.window_capacity + max(self.final_topk, self._max_selected_rows())
        self._attn_scratch = ops.Scratch(dev, ops.attention_scratch_bytes(bs, num_heads, self._attn_rows_max))

    def _max_selected_rows(self):
        """Most zone rows one attention call can be given besides the window: the full-attention regime attends every
        zone row while the sequence is shorter than the threshold."""
        return max(self.FULL_ATTENTION_THRESHOLD, self.steady_size + 2 * self.final_topk)

    def _attend(self, queries, wk, wv, n_win, *args, **kw):
        """ops.sparse_attention on the cache's own scratch (the shared, growable one for an oversized eager call)."""
        sel = args[2] if len(args) > 2 else kw.get("selected")
        rows = n_win + (sel.shape[2] if sel is not None else 0)
        scratch = self._attn_scratch if rows <= self._attn_rows_max else None
        return ops.sparse_attention(queries, wk, wv, n_win, *args, scratch=scratch, **kw)

    def check_status(self):
        """Raise if a kernel reported a bounded wait that ran out (a host synchronisation: call it between decode
        loops, not inside one)."""
        ops.check_attention_status(self._attn_scratch, self.batch_size, self.num_heads)

    # ------------------------------------------------------------------------------------------------
    # prefill
    # ------------------------------------------------------------------------------------------------
    def prefill_update_kv_cache(self, query_states, key_states, value_states, layer_idx, batch_idx):
        """key_states / value_states: [bsz, seq_len, kv_heads, 128].  bsz == 1 fills sample `batch_idx`;
        bsz == batch_size fills all samples in lockstep (same valid_start).  Returns the K/V to attend in
        the prefill itself, as the reference does (cache_hub/polar_cache.py:379-387)."""
        bsz, seq_len = key_states.shape[:2]
        assert seq_len <= self.input_length, "prompt longer than the cache was sized for"
        if bsz == 1:
            vs = self._valid_start(batch_idx)
            self._prefill_sample(key_states[0], value_states[0], layer_idx, batch_idx, vs)
            last = batch_idx + 1 == self.batch_size
        else:
            vs = self._valid_start(0)
            if batch_idx != 0:
                return key_states[:, vs:], value_states[:, vs:]
            assert bsz == self.batch_size, "lockstep prefill needs the whole batch"
            for b in range(1, bsz):
                assert self._valid_start(b) == vs, "lockstep multi-batch prefill requires one valid_start"
            for b in range(bsz):
                self._prefill_sample(key_states[b], value_states[b], layer_idx, b, vs)
            last = True
        if last:
            self.current_seq_len[layer_idx] = seq_len - vs
            if layer_idx == self.layer_num - 1:
                self.context += seq_len - vs
        return key_states[:, vs:], value_states[:, vs:]

    def _valid_start(self, b):
        vs = self.valid_start
        if isinstance(vs, (list, tuple)) or (torch.is_tensor(vs) and vs.dim() > 0):
            return int(vs[b])
        return int(vs)

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
            self._window_len[layer] = n
            self.cpu_valid_end[layer] = 0
            return
        wk[b, :, :sink] = k[:sink].transpose(0, 1)
        wv[b, :, :sink] = v[:sink].transpose(0, 1)
        wk[b, :, sink:sink + local] = k[P - local:].transpose(0, 1)
        wv[b, :, sink:sink + local] = v[P - local:].transpose(0, 1)
        self._window_len[layer] = self.steady_size
        zk = k[sink:sink + N].transpose(0, 1)   # [H, N, 128] strided view, rows 16-byte aligned
        zv = v[sink:sink + N].transpose(0, 1)
        self._append_zone(layer, b, zk, zv, 0, N, reset_counts=True)
        self.cpu_valid_end[layer] = N

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
        """Append the step's K/V row ([bs, 1, H, 128]) to the window; flush the update buffer when full."""
        pos = self._window_len[layer_idx]
        ops.append_kv(key_states, value_states, self.unified_keys_gpu[layer_idx], self.unified_values_gpu[layer_idx],
                      pos, self._dev_state[0:1] if self.device_positions else None, 0)
        self._window_len[layer_idx] = pos + 1
        self.current_seq_len[layer_idx] += 1
        if layer_idx == 0:
            self.context += 1
        if self._window_len[layer_idx] == self.window_capacity:
            self._flush(layer_idx)
        return None, None

    def _flush(self, layer):
        """Move the oldest `interval` local rows into the zone (reference: _update_polar_index,
        cache_hub/polar_cache.py:743-821, done here per layer and without blocking the host)."""
        I, sink, local = self.dynamic_update_interval, self.sink_size, self.local_size
        wk, wv = self.unified_keys_gpu[layer], self.unified_values_gpu[layer]
        N = self.cpu_valid_end[layer]
        assert N + I <= self.zone_capacity, "zone store is full"
        for b in range(self.batch_size):
            self._append_zone(layer, b, wk[b, :, sink:sink + I], wv[b, :, sink:sink + I], N, I)
        # slide [sink+I, sink+local+I) down to [sink, sink+local)
        if I < local:
            tk, tv = self._slide_tmp_k[:, :, :local], self._slide_tmp_v[:, :, :local]
            tk.copy_(wk[:, :, sink + I:sink + I + local])
            tv.copy_(wv[:, :, sink + I:sink + I + local])
            wk[:, :, sink:sink + local] = tk
            wv[:, :, sink:sink + local] = tv
        else:
            wk[:, :, sink:sink + local] = wk[:, :, sink + I:sink + I + local]
            wv[:, :, sink:sink + local] = wv[:, :, sink + I:sink + I + local]
        self.cpu_valid_end[layer] = N + I
        self._window_len[layer] = self.steady_size

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
        (cache_hub/polar_cache.py:1221-1222, :1239-1240, :1300)."""
        cand_ratio, coll_ratio = self._get_adaptive_ratios(N)
        tiers = [int(math.ceil(N * coll_ratio * r)) for r in TIER_RATIOS]
        C = max(1, int(math.ceil(N * cand_ratio)))
        return tiers, C, min(self.final_topk, C)

    def compute(self, queries, layer_idx):
        """Decode attention of one token: queries [bs, 1, num_heads, 128] -> [bs, 1, num_heads, 128]."""
        queries = queries.contiguous()
        self._wait_offload(layer_idx)
        N = self.cpu_valid_end[layer_idx]
        n_win = self._window_len[layer_idx]
        total = self.current_seq_len[layer_idx]
        wk, wv = self.unified_keys_gpu[layer_idx], self.unified_values_gpu[layer_idx]
        sk, sv = self._store_k[layer_idx], self._store_v[layer_idx]
        full = total < max(self.FULL_ATTENTION_THRESHOLD, self.steady_size + 2 * self.final_topk) or N <= 0
        if full:  # cache_hub/polar_cache.py:1033-1045: attend everything
            if N <= 0:
                return self._attend(queries, wk, wv, n_win)
            if self._all_rows is None or self._all_rows.shape[-1] < N:
                self._all_rows = torch.arange(self.zone_capacity, device=self.device).expand(
                    self.batch_size, self.kv_head, -1).contiguous()
            sel = self._all_rows[:, :, :N].contiguous() if N != self._all_rows.shape[-1] else self._all_rows
            return self._attend(queries, wk, wv, n_win, sk, sv, sel)
        tiers, C, K = self.retrieval_plan(N)
        final, _ = ops.retrieve(queries, self.srht_diagonal_signs, self._mag_centers,
                                self.codebook_gpu[layer_idx][:, :, :, :N], self.key_block_weight_gpu[layer_idx][:, :, :, :N],
                                self.key_4bit_packed_gpu[layer_idx][:, :, :, :N, :], self.cluster_key_counts_gpu[layer_idx],
                                tiers, C, K, scratch=self._retrieve_scratch)
        self.last_topk_indices = final
        if self.device_positions:  # rows = (window length at step start) + this step's row, read on the device
            return self._attend(queries, wk, wv, self.window_capacity, sk, sv, final,
                                n_window_dev=self._dev_state[0:1], n_window_add=1)
        return self._attend(queries, wk, wv, n_win, sk, sv, final)

    # ------------------------------------------------------------------------------------------------
    # support for replaying a captured decode step
    # ------------------------------------------------------------------------------------------------
    def next_step_flushes(self) -> bool:
        """True when the next appended token fills the update buffer (that step must run eagerly)."""
        return self._window_len[0] + 1 >= self.window_capacity

    def sync_device_state(self):
        """Copy the host-side window length to the device word read when device_positions is set."""
        self._dev_state[0] = self._window_len[0]

    def advance_device_step(self):
        """Device-side end of a step: one more row in the window (a launch, so it is captured with the step)."""
        self._dev_state[0:1] += 1

    def host_state(self):
        return (list(self._window_len), list(self.current_seq_len), self.context, list(self.cpu_valid_end))

    def set_host_state(self, st):
        self._window_len, self.current_seq_len, self.context, self.cpu_valid_end = list(st[0]), list(st[1]), st[2], list(st[3])

    def host_state_after_flushes(self, j):
        """The host state right after the j-th flush from now (None when the zone cannot grow that far): what a
        step captured ahead of time needs, since capturing only records launch arguments."""
        n = self.cpu_valid_end[0] + j * self.dynamic_update_interval
        if n > self.zone_capacity:
            return None
        L = self.layer_num
        return ([self.steady_size] * L, list(self.current_seq_len), self.context, [n] * L)

    def note_replayed_step(self):
        """Host-side bookkeeping of one decode step that ran as a graph replay."""
        for l in range(self.layer_num):
            self._window_len[l] += 1
            self.current_seq_len[l] += 1
        self.context += 1

    def sync(self, layer_idx, batch_idx):
        """Order the current stream after the layer's bulk offload (cache_hub/polar_cache.py:617-639).  The
        reference blocks the host here; a stream-side wait is enough because every consumer is a kernel."""
        self._wait_offload(layer_idx)
        return None
