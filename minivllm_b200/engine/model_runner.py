"""Model runner: step metadata on the GPU, KV-cache allocation, eager prefill
and CUDA-graph decode around the attention path.

Same responsibilities and method names as the reference's
src/myvllm/engine/model_runner.py (`prepare_prefill` :180, `prepare_decode`
:231, `run_model` :267, `run` :298, `capture_cudagraph` :317,
`allocate_kv_cache` :140), redesigned:
  * metadata comes from device-resident sequence state (engine/metadata.py);
    the host uploads slot ids only, never slot_mapping / block tables;
  * one captured graph per padded batch size holds the WHOLE decode step:
    metadata kernel, every layer, LM head, sampling and the write-back of the
    sampled token into the device state — a replay needs no host-built tensor
    and its only host traffic is the batch of sampled token ids coming back;
  * tensor parallelism is SPMD: every rank runs this same runner on its own
    GPU and makes the same scheduling decisions from the same sampled tokens,
    so the reference's shared-memory RPC to worker processes is not needed.
    The only collectives are the NCCL all-reduces inside the model.
"""
import math

import torch
import torch.distributed as dist

from ..layers.attention import _error_word
from ..utils.context import get_context, reset_context, set_context
from .metadata import SequenceStateTable
from ..layers.sampler import greedy_tokens, sampled_tokens
from .qwen3 import Qwen3Config, Qwen3ForCausalLM


def _cfg(config, *names, default=None):
    for n in names:
        if n in config:
            return config[n]
    return default


class ModelRunner:
    def __init__(self, config: dict, rank: int = 0, world_size: int = None, device=None, model=None):
        self.config = config
        self.rank = rank
        self.world_size = world_size if world_size is not None else config.get("world_size", 1)
        self.block_size = config.get("block_size", 256)
        self.enforce_eager = config.get("enforce_eager", False)
        self.max_num_seqs = _cfg(config, "max_num_seqs", "max_num_sequences", default=16)
        self.max_num_batched_tokens = _cfg(config, "max_num_batched_tokens", "max_num_batch_tokens", default=1024)
        self.max_model_len = _cfg(config, "max_model_length", "max_position", default=4096)
        self.dtype = config.get("dtype", torch.bfloat16)
        self.device = torch.device(device if device is not None else f"cuda:{torch.cuda.current_device()}")
        self.greedy = config.get("greedy", False)
        # "int8": per-token-per-head symmetric int8 KV cache with fp16 scales (no counterpart in the reference)
        self.kv_int8 = config.get("kv_cache_dtype", None) == "int8"
        if self.kv_int8 and config.get("enable_prefix_caching", False):
            raise ValueError("kv_cache_dtype='int8' cannot be combined with prefix caching: the prefix-aware prefill "
                             "kernel reads fp16/bf16 caches only")
        mcfg = Qwen3Config.from_dict(config)
        mcfg.max_position = max(mcfg.max_position, self.max_model_len)
        self.model_cfg = mcfg
        self.model = model if model is not None else Qwen3ForCausalLM(
            mcfg, tp_rank=rank, tp_size=self.world_size, dtype=self.dtype, device=self.device,
            seed=config.get("seed", 0))
        self.comm, self.comm_note = None, "single rank"
        if self.world_size > 1:
            self._attach_communicator()
        # prefill_streams=2 (the default under tensor parallelism): two prefill waves in flight on two streams, so
        # that one wave's all-reduces (bound by the link) run beside the other wave's GEMMs.  Each stream has a
        # communicator of its own whose calls take the copy-engine form (layers/allreduce.py, staged=True): the
        # fused kernel needs most SMs to fill the link, the copy engines need none; the sums and roundings are
        # the same, so the tokens are those of the one-stream engine.  Greedy runs only: a sampled run advances
        # one step counter in stream order.
        self.prefill_lanes, self._prefill_at = [], 0
        want = int(config.get("prefill_streams", 2 if self.comm is not None else 1))
        if want >= 2 and self.greedy and self.device.type == "cuda":
            lanes = []
            for _ in range(2):
                comm = self._new_communicator(staged=True) if self.comm is not None else None
                if self.comm is not None and comm is None:
                    break
                lanes.append((torch.cuda.Stream(device=self.device), comm))
            if len(lanes) == 2:
                self.prefill_lanes = lanes
            else:
                for _, comm in lanes:
                    if comm is not None:
                        comm.close()
        self.error_word = _error_word(self.device)
        self.max_blocks_per_seq = math.ceil(self.max_model_len / self.block_size)
        # one spare slot: padded rows of a captured batch point at it
        self.num_slots = self.max_num_seqs + 1
        self.pad_slot = self.max_num_seqs
        self.state = SequenceStateTable(self.num_slots, self.max_blocks_per_seq, self.block_size, self.device)
        # temperature sampling: same seed on every rank, a step counter in device memory that the decode graph
        # advances itself
        self.sample_seed = int(config.get("sample_seed", 1234))
        self.sample_step = torch.zeros(1, dtype=torch.int64, device=self.device)
        self.graphs, self.graph_vars = {}, None
        self.decode_workspace = None
        self._stage, self._stage_at, self._stage_dev = None, 0, None
        self._readback, self._readback_at = None, 0
        self.allocate_kv_cache()
        if not self.enforce_eager:
            self.capture_cudagraph()

    # ------------------------------------------------------------------ memory ---
    def kv_block_bytes(self):
        c = self.model_cfg
        rows = self.block_size * 2 * c.num_layers * (c.num_kv_heads // self.world_size)
        if self.kv_int8:
            return rows * (c.head_dim + 2)             # int8 codes + one fp16 scale per row
        return rows * c.head_dim * torch.empty((), dtype=self.dtype).element_size()

    def allocate_kv_cache(self):
        """One pool (2, layers, blocks, block_size, kv_heads/tp, head_dim); every module that has
        `k_cache` and `v_cache` attributes gets its layer's views (the reference's duck typing,
        model_runner.py:162-168)."""
        c = self.model_cfg
        if "num_kv_blocks" in self.config:
            num_blocks = int(self.config["num_kv_blocks"])
        else:
            free, _ = torch.cuda.mem_get_info(self.device)
            util = self.config.get("gpu_memory_utilization", 0.9)
            reserve = self.config.get("activation_reserve_bytes", self._activation_reserve())
            num_blocks = int((free * util - reserve) // self.kv_block_bytes())
            if self.world_size > 1:  # every rank must agree on the pool size: the scheduler state is replicated
                t = torch.tensor([num_blocks], device=self.device, dtype=torch.int64)
                dist.all_reduce(t, op=dist.ReduceOp.MIN)
                num_blocks = int(t.item())
        assert num_blocks >= 1, f"not enough memory for one KV block on rank {self.rank}"
        self.num_kv_blocks = num_blocks
        kvh = c.num_kv_heads // self.world_size
        self.kv_cache = torch.zeros(2, c.num_layers, num_blocks, self.block_size, kvh, c.head_dim,
                                    dtype=torch.int8 if self.kv_int8 else self.dtype, device=self.device)
        self.kv_scale = torch.zeros(2, c.num_layers, num_blocks, self.block_size, kvh, dtype=torch.float16,
                                    device=self.device) if self.kv_int8 else None
        layer = 0
        for module in self.model.modules():
            if hasattr(module, "k_cache") and hasattr(module, "v_cache"):
                module.k_cache = self.kv_cache[0, layer]
                module.v_cache = self.kv_cache[1, layer]
                if self.kv_int8:
                    module.k_scale, module.v_scale = self.kv_scale[0, layer], self.kv_scale[1, layer]
                layer += 1
        assert layer == c.num_layers

    def _activation_reserve(self):
        """Peak activation bytes of the largest prefill wave (logits of the last tokens included), estimated
        from shapes instead of the reference's warm-up run."""
        c, t = self.model_cfg, self.max_num_batched_tokens
        per_tok = (c.hidden_size * 6 + (c.num_heads + 2 * c.num_kv_heads) * c.head_dim * 3 // self.world_size +
                   3 * c.intermediate_size * 2 // self.world_size) * 4
        return t * per_tok + self.max_num_seqs * c.vocab_size * 8 + (2 << 30)

    # ---------------------------------------------------------------- metadata ---
    def _sync_tables(self, seqs):
        """Block-table entries the device rows do not hold yet (new sequences, sequences that grew)."""
        upd = []
        for s in seqs:
            if s.synced_blocks == 0 and s.block_table:
                row = list(s.block_table) + [-1] * (self.max_blocks_per_seq - len(s.block_table))
                upd.extend((s.slot, i, b) for i, b in enumerate(row))
            else:
                upd.extend((s.slot, i, s.block_table[i]) for i in range(s.synced_blocks, len(s.block_table)))
            s.synced_blocks = len(s.block_table)
        self.state.update_tables(upd)

    def prepare_prefill(self, seqs):
        self._sync_tables(seqs)
        ids = [t for s in seqs for t in s.token_ids[s.num_cached_tokens:]]
        input_ids = torch.tensor(ids, dtype=torch.int64).pin_memory().to(self.device, non_blocking=True)
        meta = self.state.build_prefill([s.slot for s in seqs], [len(s) for s in seqs],
                                        [s.num_cached_tokens for s in seqs])
        tables = None
        if any(s.num_cached_tokens for s in seqs):
            # a prefix hit: attention must read keys through the block tables (the reference sets them too,
            # model_runner.py:209-215, but its kernel never uses them)
            slots = torch.tensor([s.slot for s in seqs], dtype=torch.int64).pin_memory().to(self.device,
                                                                                             non_blocking=True)
            tables = self.state.tables.index_select(0, slots)
        set_context(True, meta["cu_seqlens_q"], meta["cu_seqlens_k"], meta["max_seqlen_q"], meta["max_seqlen_k"],
                    meta["slot_mapping"], None, tables, positions=meta["positions"],
                    last_token_index=meta["last_token_index"])
        return input_ids

    def _attach_communicator(self):
        """The fused all-reduce + residual + RMSNorm over NVLink peer memory (layers/allreduce.py) replaces the
        NCCL all-reduces of the model.  If the peer mapping cannot be set up (every rank learns it at the same
        point), the model keeps NCCL and says so in `comm_note`."""
        if not self.config.get("custom_allreduce", True):
            self.comm_note = "NCCL all-reduce (custom_allreduce=False)"
            return
        comm = self._new_communicator()
        if comm is not None:
            self.comm, self.model.comm = comm, comm
            self.comm_note = "fused all-reduce + residual + RMSNorm kernel over NVLink peer memory"
        else:
            self.comm_note = "NCCL all-reduce (peer-memory communicator unavailable: %s)" % self._comm_error
            if self.rank == 0:
                print("minivllm_b200: " + self.comm_note, flush=True)

    def _new_communicator(self, staged=False):
        """A peer-memory communicator for this rank, or None on EVERY rank if any rank could not set it up."""
        from ..layers.allreduce import TPCommunicator
        err, comm = "", None
        try:
            comm = TPCommunicator(self.rank, self.world_size, self.max_num_batched_tokens, self.model_cfg.hidden_size,
                                  self.dtype, self.device, timeout_ms=self.config.get("comm_timeout_ms", 5000),
                                  staged=staged)
        except Exception as e:  # noqa: BLE001 - reported, and agreed on by all ranks below
            err = f"{type(e).__name__}: {e}"
        ok = torch.tensor([0 if err else 1], device=self.device, dtype=torch.int32)
        dist.all_reduce(ok, op=dist.ReduceOp.MIN)
        if int(ok.item()) == 1:
            return comm
        if comm is not None:
            comm.close()
        self._comm_error = err or "failed on another rank"
        return None

    def _upload_slots(self, seqs, slots_buf, n_active_buf):
        """Slot ids of the batch (padding rows point at the spare slot) and the live count: one pinned staging
        row out of a small ring, one H2D copy."""
        bp = slots_buf.shape[0]
        if self._stage is None:
            self._stage = [torch.empty(self.max_num_seqs + 1, dtype=torch.int32).pin_memory() for _ in range(4)]
            self._stage_dev = torch.empty(self.max_num_seqs + 1, dtype=torch.int32, device=self.device)
        host = self._stage[self._stage_at % len(self._stage)]
        self._stage_at += 1
        n = len(seqs)
        host[:n] = torch.tensor([s.slot for s in seqs], dtype=torch.int32)
        host[n:bp] = self.pad_slot
        host[bp] = n
        dev = self._stage_dev[:bp + 1]
        dev.copy_(host[:bp + 1], non_blocking=True)
        slots_buf.copy_(dev[:bp])
        n_active_buf.copy_(dev[bp:])

    def prepare_decode(self, seqs, bufs=None, slots_buf=None, n_active_buf=None):
        """Eager form: allocates the step's buffers; the graph path passes its static ones."""
        self._sync_tables(seqs)
        if bufs is None:
            bp = len(seqs)
            bufs = self.state.new_decode_buffers(bp)
            slots_buf = torch.empty(bp, dtype=torch.int32, device=self.device)
            n_active_buf = torch.empty(1, dtype=torch.int32, device=self.device)
        self._upload_slots(seqs, slots_buf, n_active_buf)
        self.state.build_decode(slots_buf, n_active_buf, bufs)
        self._set_decode_context(bufs)
        return bufs["input_ids"], slots_buf

    def _set_decode_context(self, bufs):
        set_context(False, None, None, 0, 0, bufs["slot_mapping"], bufs["context_lens"], bufs["block_tables"],
                    positions=bufs["positions"], decode_workspace=self.decode_workspace)

    # ---------------------------------------------------------------- sampling ---
    def next_tokens(self, hidden, temperatures=None):
        """hidden states -> sampled token ids.  Each rank multiplies by its slice of the vocabulary only and
        reduces it to one 64-bit key per row (layers/sampler.py): the row maximum when greedy, the best
        exponential-race score (the reference's sampler, src/myvllm/layers/sampler.py:15-19, without its softmax)
        when sampling with temperatures -- rows with temperature 0 are greedy.  Ranks merge the keys by MAX
        instead of gathering or replicating the 151,936-wide logits, and end with identical tokens: the race's
        noise depends on (seed, step, row, global column) only."""
        vocab = self.model.lm_head.shape[0]
        shard = self.world_size > 1 and vocab % self.world_size == 0
        if shard:
            logits = self.model.compute_logits(hidden, (self.rank, self.world_size))
            offset, world = self.rank * (vocab // self.world_size), self.world_size
        else:
            logits = self.model.compute_logits(hidden)
            offset, world = 0, 1
        if self.greedy or temperatures is None:
            return greedy_tokens(logits, offset, None, world)
        tokens = sampled_tokens(logits, temperatures, self.sample_seed, self.sample_step, offset, None, world)
        self.sample_step.add_(1)
        return tokens

    # --------------------------------------------------------------------- run ---
    @torch.inference_mode()
    def run_model(self, input_ids, is_prefill):
        """Hidden states of the rows that get a next token (last token of each sequence in prefill)."""
        return self.model(input_ids)

    def run(self, seqs, is_prefill):
        """One model step, synchronously: sampled token ids of `seqs` as a Python list."""
        return self.finish(self.launch(seqs, is_prefill))

    @torch.inference_mode()
    def launch(self, seqs, is_prefill):
        """Enqueues one model step and the device->host copy of its result; returns a handle for `finish`.
        Nothing here waits for the GPU."""
        if is_prefill and self.prefill_lanes:
            return self._launch_prefill_lane(seqs)
        main = torch.cuda.current_stream() if self.device.type == "cuda" else None
        for stream, _ in self.prefill_lanes:         # a step on the main stream sees every wave launched so far
            main.wait_stream(stream)
        temps = None
        if not self.greedy:
            temps = torch.tensor([s.temperature for s in seqs], dtype=torch.float32).pin_memory().to(
                self.device, non_blocking=True)
        n = len(seqs)
        if is_prefill:
            result = self._prefill_body(seqs, temps)
        elif self.enforce_eager or not self.graphs:
            input_ids, slots_buf = self.prepare_decode(seqs)
            tokens = self.next_tokens(self.run_model(input_ids, False), temps)
            self.state.last_token.index_copy_(0, slots_buf.long(), tokens)
            result = torch.cat([tokens, self.error_word.to(torch.int64)])
        else:
            result = self._replay(seqs, temps)      # (max_num_seqs + 1,): tokens, then the error word
        reset_context()
        if self._readback is None:
            self._readback = [torch.empty(max(self.max_num_seqs, self.max_num_batched_tokens) + 1,
                                          dtype=torch.int64).pin_memory() for _ in range(4)]
        return self._read_back(result, n)

    def _read_back(self, result, n):
        host = self._readback[self._readback_at % len(self._readback)][:result.numel()]
        self._readback_at += 1
        host.copy_(result, non_blocking=True)        # the step's only device->host read
        done = torch.cuda.Event()
        done.record()
        return host, done, n

    def _prefill_body(self, seqs, temps):
        input_ids = self.prepare_prefill(seqs)
        tokens = self.next_tokens(self.run_model(input_ids, True), temps)
        slots = torch.tensor([s.slot for s in seqs], dtype=torch.int64).pin_memory().to(self.device,
                                                                                         non_blocking=True)
        self.state.last_token.index_copy_(0, slots, tokens)
        return torch.cat([tokens, self.error_word.to(torch.int64)])

    def _launch_prefill_lane(self, seqs):
        """A prefill wave on the next of the two side streams.  The wave before it may still be running on the
        other one: the waves touch different sequences (rows of the state tables, cache blocks), every tensor of
        a wave is allocated on its stream, and a wave that reads cached blocks waits for the other stream first
        (the blocks may have been written there)."""
        lane = self._prefill_at % len(self.prefill_lanes)
        self._prefill_at += 1
        stream, comm = self.prefill_lanes[lane]
        main = torch.cuda.current_stream()
        stream.wait_stream(main)
        if any(s.num_cached_tokens for s in seqs):
            for other, _ in self.prefill_lanes:
                if other is not stream:
                    stream.wait_stream(other)
        if comm is not None:
            self.model.comm = comm
        try:
            with torch.cuda.stream(stream):
                result = self._prefill_body(seqs, None)
                reset_context()
                if self._readback is None:
                    self._readback = [torch.empty(max(self.max_num_seqs, self.max_num_batched_tokens) + 1,
                                                  dtype=torch.int64).pin_memory() for _ in range(4)]
                return self._read_back(result, len(seqs))
        finally:
            if comm is not None:
                self.model.comm = self.comm

    def finish(self, handle):
        """Waits for a launched step; raises if a kernel wait of the step ran out of time."""
        host, done, n = handle
        done.synchronize()
        code = int(host[-1])
        if code:
            self.error_word.zero_()
            raise RuntimeError(
                f"a bounded wait inside a kernel ran out of time (error word {code:#x}): "
                + ("a tensor-parallel peer did not arrive; the communicator must be reset on every rank"
                   if code >= 0x100 else "prefill attention pipeline") + "; the step's tokens are not valid")
        return host[:n].tolist()

    # ------------------------------------------------------------------ graphs ---
    def _decode_body(self, v, bp):
        """The whole decode step on static buffers; captured once per padded batch size."""
        bufs = {k: t[:bp] for k, t in v["bufs"].items()}
        self.state.build_decode(v["slots"][:bp], v["n_active"], bufs)
        self._set_decode_context(bufs)
        tokens = self.next_tokens(self.model(bufs["input_ids"]), None if self.greedy else v["temps"][:bp])
        v["tokens"][:bp].copy_(tokens)
        v["tokens"][self.max_num_seqs:].copy_(self.error_word)
        self.state.last_token.index_copy_(0, v["slots"][:bp].long(), tokens)

    @torch.inference_mode()
    def capture_cudagraph(self):
        max_bs = self.max_num_seqs
        v = dict(bufs=self.state.new_decode_buffers(max_bs),
                 slots=torch.full((max_bs,), self.pad_slot, dtype=torch.int32, device=self.device),
                 n_active=torch.zeros(1, dtype=torch.int32, device=self.device),
                 temps=torch.ones(max_bs, dtype=torch.float32, device=self.device),
                 tokens=torch.zeros(max_bs + 1, dtype=torch.int64, device=self.device))
        c = self.model_cfg
        from .. import _cabi
        need = _cabi.lib().mv_paged_decode_workspace_bytes(max_bs, c.num_heads // self.world_size,
                                                           c.num_kv_heads // self.world_size, c.head_dim,
                                                           self.max_blocks_per_seq, self.block_size)
        self.decode_workspace = torch.zeros(max(need, 1), dtype=torch.uint8, device=self.device)
        sizes = [b for b in [1, 2, 4, 8] if b <= max_bs] + list(range(16, max_bs + 1, 16))
        if max_bs not in sizes:
            sizes.append(max_bs)
        self.graph_vars, pool = v, None
        # n_active = 0 during warm-up and capture: every row is padding, no sequence state is touched
        for bp in sorted(set(sizes), reverse=True):
            self._decode_body(v, bp)               # warm-up (also resolves lazy initialisation)
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, pool=pool):
                self._decode_body(v, bp)
            pool = pool or g.pool()
            self.graphs[bp] = g
        torch.cuda.synchronize()
        reset_context()

    def _replay(self, seqs, temps):
        bs = len(seqs)
        bp = next(b for b in sorted(self.graphs) if b >= bs)
        v = self.graph_vars
        self._sync_tables(seqs)
        self._upload_slots(seqs, v["slots"][:bp], v["n_active"])
        if temps is not None:
            v["temps"][:bs].copy_(temps)
        self.graphs[bp].replay()
        return v["tokens"]

    def exit(self):
        torch.cuda.synchronize()
        self.graphs, self.graph_vars = {}, None
        if self.comm is not None:
            self.model.comm = None
            if self.world_size > 1:
                dist.barrier()           # no rank unmaps while a peer may still be inside a kernel
            for _, comm in self.prefill_lanes:
                if comm is not None:
                    comm.close()
            self.prefill_lanes = []
            self.comm.close()
            self.comm = None
        torch.cuda.synchronize()
