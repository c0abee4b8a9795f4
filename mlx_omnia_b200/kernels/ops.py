"""The operations the parts are written in, each one a launch of this package's own
CUDA kernels (sources under `csrc/`). There is no other implementation behind these
functions: on a machine without a CUDA device or without nvcc they raise.

Conventions: tensors are contiguous CUDA tensors; `dtype` is float32 or bfloat16 and
names the element type of activations, matrices and cache pages; the residual stream
`x` and all logits are float32; integer metadata is int32 except `slot_mapping`
(int64). Functions return new tensors unless they say "in place".
"""

from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_longlong, c_void_p

import dataclasses
from dataclasses import dataclass

import numpy as np
import torch

from mlx_omnia_b200.csrc.build import load_library
from mlx_omnia_b200.parts.base import KVView, StepContext

_DTYPE_CODE = {torch.float32: 0, torch.bfloat16: 1}

ERROR_BITS = {1: "a token id outside the embedding table", 2: "a cache slot outside the page pool",
              4: "a block-table entry outside the page pool", 8: "a bounded wait inside a kernel ran out",
              16: "a work list asked a kernel for what it does not do"}


class KernelError(RuntimeError):
    """A kernel launch failed, or a kernel reported bad indices."""


_functions: dict[str, ctypes._CFuncPtr] = {}
_error_words: dict[int, torch.Tensor] = {}


def _function(library: str, name: str, argtypes: list, defines: dict | None = None):
    key = f"{library}:{name}:{sorted((defines or {}).items())}"
    fn = _functions.get(key)
    if fn is None:
        fn = getattr(load_library(library, defines), name)
        fn.argtypes = argtypes
        fn.restype = c_int
        _functions[key] = fn
    return fn


def _ptr(t: torch.Tensor | None) -> int | None:
    return None if t is None else t.data_ptr()


def _stream() -> int:
    """The current stream's handle (the raw query: `torch.cuda.current_stream()` builds a Python
    object and costs 3 us, which a step of 230 launches pays 230 times)."""
    return torch._C._cuda_getCurrentRawStream(torch.cuda.current_device())


launches = 0
"""How many launches of this package's own kernels this process has issued (a call that
launches two kernels counts once; replayed CUDA graphs add what their capture recorded)."""


def _check(code: int, what: str) -> None:
    global launches
    launches += 1
    if code != 0:
        raise KernelError(f"{what}: CUDA error {code} at launch (bad sizes for this kernel, or an earlier fault)")


def _code(dtype: torch.dtype) -> int:
    try:
        return _DTYPE_CODE[dtype]
    except KeyError:
        raise KernelError(f"kernels take float32 or bfloat16, not {dtype}") from None


def error_word(device: torch.device) -> torch.Tensor:
    """The int32 word that kernels OR their index-check failures into."""
    index = device.index if device.index is not None else torch.cuda.current_device()
    word = _error_words.get(index)
    if word is None:
        word = torch.zeros(1, dtype=torch.int32, device=device)
        _error_words[index] = word
    return word


def raise_on_error(device: torch.device) -> None:
    """Read the error word (a device sync) and raise if any kernel flagged bad indices."""
    word = error_word(device)
    bits = int(word.item())
    if bits:
        word.zero_()
        # A kernel that gave up may have left its tickets half drawn: the buffers that their users
        # are to leave zero are zero again for the next launch.
        for key in _zeroed:
            if key[0] == (device.index or 0):
                _scratch[key].zero_()
        raise KernelError("kernel index check failed: " + "; ".join(m for b, m in ERROR_BITS.items() if bits & b))


def require_cuda() -> None:
    if not torch.cuda.is_available():
        raise KernelError("mlx_omnia_b200 runs on a CUDA device (sm_100a) only; none is visible")


_sm_counts: dict[int, int] = {}


def sm_count(device: torch.device | None = None) -> int:
    """How many SMs `device` (the current one when None) has; asked once per device. Plans that
    count waves or shares of the GPU are made from this."""
    index = torch.cuda.current_device() if device is None or device.index is None else device.index
    count = _sm_counts.get(index)
    if count is None:
        count = _sm_counts[index] = torch.cuda.get_device_properties(index).multi_processor_count
    return count


# ------------------------------------------------------------------------------------


def embed_rmsnorm(ids: torch.Tensor, table: torch.Tensor, eps: float | None) -> torch.Tensor:
    """x[t] = table[ids[t]], RMS-normalised without a weight when `eps` is given. -> float32."""
    tokens, (vocab, hidden) = ids.shape[0], table.shape
    x = torch.empty(tokens, hidden, dtype=torch.float32, device=table.device)
    fn = _function("elementwise", "omnia_embed_rmsnorm",
                   [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_int, c_int, c_void_p, c_void_p])
    _check(fn(_ptr(ids), _ptr(table), _ptr(x), tokens, hidden, vocab, 0.0 if eps is None else eps,
              int(eps is not None), _code(table.dtype), _ptr(error_word(table.device)), _stream()), "embed_rmsnorm")
    return x


def embed_pair(step: StepContext, table: torch.Tensor, pairs: torch.Tensor, prev: torch.Tensor, scale: float,
               mul_prev: int, mul_cur: int) -> torch.Tensor:
    """x[t] = table[id_t] * scale + pairs[(id_before * mul_prev + id_t * mul_cur) mod buckets], with
    buckets = rows of `pairs` - 1 and the extra last row for a request's first token. The token before a
    portion's first one is read from `prev` (int32 [slots], by state slot), which then receives the
    portion's last token. -> float32 [tokens, hidden]."""
    tokens, (vocab, hidden) = step.token_ids.shape[0], table.shape
    x = torch.empty(tokens, hidden, dtype=torch.float32, device=table.device)
    fn = _function("elementwise", "omnia_embed_pair",
                   [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int,
                    c_int, c_longlong, c_longlong, c_longlong, c_float, c_int, c_void_p, c_void_p])
    _check(fn(_ptr(step.token_ids), _ptr(step.positions), _ptr(step.cu_seqlens), _ptr(step.state_slots),
              step.num_seqs, _ptr(table), _ptr(pairs), _ptr(prev), _ptr(x), tokens, hidden, vocab,
              pairs.shape[0] - 1, mul_prev, mul_cur, scale, _code(table.dtype), _ptr(error_word(table.device)),
              _stream()), "embed_pair")
    return x


def rounded_rows(x: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    """The float32 residual `x` as activations of `dtype` (x itself when that is float32)."""
    if dtype == torch.float32:
        return x
    h = torch.empty(x.shape, dtype=dtype, device=x.device)
    fn = _function("elementwise", "omnia_round_rows", [c_void_p, c_void_p, c_longlong, c_int, c_void_p])
    _check(fn(_ptr(x), _ptr(h), x.numel(), _code(dtype), _stream()), "round_rows")
    return h


def rmsnorm(x: torch.Tensor, weight: torch.Tensor | None, eps: float, dtype: torch.dtype) -> torch.Tensor:
    """h = x * rsqrt(mean x^2 + eps) * weight, x float32 [rows, hidden] -> `dtype`."""
    rows, hidden = x.shape
    h = torch.empty(rows, hidden, dtype=dtype, device=x.device)
    fn = _function("elementwise", "omnia_rmsnorm", [c_void_p, c_void_p, c_void_p, c_int, c_int, c_float, c_int, c_void_p])
    _check(fn(_ptr(x), _ptr(weight), _ptr(h), rows, hidden, eps, _code(dtype), _stream()), "rmsnorm")
    return h


def add_rmsnorm(x: torch.Tensor, branch: torch.Tensor, branch_weight: torch.Tensor | None,
                branch_eps: float | None, out_weight: torch.Tensor | None, out_eps: float | None,
                rounded: bool = False) -> torch.Tensor | None:
    """x += norm_b(branch) in place (float32), then h = norm_o(x) in branch's dtype.
    `branch_eps is None` adds the branch as it is; `out_eps is None` returns no h, unless `rounded`:
    h is then the new x itself in branch's dtype (for a part that reads the residual unnormed)."""
    rows, hidden = x.shape
    if rounded and out_eps is None:
        h = torch.empty_like(branch)
        fn = _function("elementwise", "omnia_add_rmsnorm",
                       [c_void_p, c_void_p, c_void_p, c_float, c_int, c_void_p, c_float, c_int, c_void_p, c_int, c_int, c_int, c_void_p])
        _check(fn(_ptr(x), _ptr(branch), _ptr(branch_weight), branch_eps or 0.0, int(branch_eps is not None),
                  None, 0.0, 2, _ptr(h), rows, hidden, _code(branch.dtype), _stream()), "add_rmsnorm")
        return h
    h = torch.empty_like(branch) if out_eps is not None else None
    fn = _function("elementwise", "omnia_add_rmsnorm",
                   [c_void_p, c_void_p, c_void_p, c_float, c_int, c_void_p, c_float, c_int, c_void_p, c_int, c_int, c_int, c_void_p])
    _check(fn(_ptr(x), _ptr(branch), _ptr(branch_weight), branch_eps or 0.0, int(branch_eps is not None),
              _ptr(out_weight), out_eps or 0.0, int(out_eps is not None), _ptr(h), rows, hidden,
              _code(branch.dtype), _stream()), "add_rmsnorm")
    return h


def qk_norm_rope_store(proj: torch.Tensor, q_col: int, k_col: int, v_col: int, nq: int, nkv: int, d: int,
                       eps: float | None, inv_freq: torch.Tensor | None, positions: torch.Tensor,
                       kv: KVView | None) -> torch.Tensor:
    """Per head of the projected rows: weightless RMS (q, k), rotation of the first
    2 * len(inv_freq) dims, q out as [tokens, nq, d], k and v into the cache pages.
    With `kv` None or not writing, only q is produced."""
    tokens, stride = proj.shape
    q = torch.empty(tokens, nq, d, dtype=proj.dtype, device=proj.device)
    store = kv is not None and kv.writes
    rot = 0 if inv_freq is None else 2 * inv_freq.shape[0]
    fn = _function("elementwise", "omnia_qk_norm_rope_store",
                   [c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_void_p, c_int, c_void_p,
                    c_void_p, c_void_p, c_void_p, c_int, c_longlong, c_int, c_int, c_void_p, c_void_p])
    _check(fn(_ptr(proj), stride, q_col, k_col, v_col, nq, nkv if store else 0, d, -1.0 if eps is None else eps,
              _ptr(inv_freq), rot, _ptr(positions), _ptr(kv.slot_mapping) if store else None, _ptr(q),
              _ptr(kv.pages) if store else None, kv.page_size if store else 1,
              kv.pages.shape[0] * kv.page_size if store else 0, tokens, _code(proj.dtype),
              _ptr(error_word(proj.device)), _stream()), "qk_norm_rope_store")
    return q


def kv_layout(kv: KVView) -> tuple[int, int, int, int, int, int]:
    """(address of the keys of page 0, of its values, elements from a page to the next, key/value
    heads, key width, value width) of an attention cache: two rows `(heads, width)` a position, of
    equal widths (pages [num_pages, 2, heads, page_size, width]) or not (pages [num_pages, elements])."""
    (nkv, dk), (_, dv) = kv.spec.rows if kv.spec is not None else ((kv.pages.shape[2], kv.pages.shape[4]),) * 2
    item = kv.pages.element_size()
    base = kv.pages.data_ptr()
    return base, base + nkv * dk * kv.page_size * item, nkv * (dk + dv) * kv.page_size, nkv, dk, dv


def qkv_prepare(proj: torch.Tensor, q_col: int, k_col: int, v_col: int, nq: int, dk: int, bias: torch.Tensor | None,
                q_weight: torch.Tensor | None, k_weight: torch.Tensor | None, eps: float | None,
                inv_freq: torch.Tensor | None, positions: torch.Tensor, kv: KVView, store: bool,
                whole: bool = False, interleaved: bool = False) -> torch.Tensor:
    """Per head of the projected rows: bias (the whole row's, [columns]), RMS norm with a weight of the
    head's size (q and k), rotation of the first 2 * len(inv_freq) dims in half-split pairs; q out as
    [tokens, nq, dk], and with `store` the keys and the values (of a width of their own) into the cache.
    `whole`: the norm is one root mean square over all heads of q at once (and one over all heads of k),
    its weights of the whole projection's size ([nq * dk], [nkv * dk]); `interleaved`: the rotation pairs
    dims (2i, 2i + 1) instead of (i, i + half)."""
    tokens, stride = proj.shape
    k_ptr, v_ptr, page_stride, nkv, kdim, dv = kv_layout(kv)
    if kdim != dk:
        raise KernelError(f"the cache keeps keys of {kdim}, the mixer makes keys of {dk}")
    q = torch.empty(tokens, nq, dk, dtype=proj.dtype, device=proj.device)
    rot = 0 if inv_freq is None else 2 * inv_freq.shape[0]
    fn = _function("elementwise", "omnia_qkv_prepare",
                   [c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p,
                    c_float, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_longlong, c_int,
                    c_longlong, c_int, c_int, c_int, c_int, c_void_p, c_void_p])
    _check(fn(_ptr(proj), stride, q_col, k_col, v_col, nq, nkv if store else 0, dk, dv, _ptr(bias), _ptr(q_weight),
              _ptr(k_weight), -1.0 if eps is None else eps, _ptr(inv_freq), rot, _ptr(positions),
              _ptr(kv.slot_mapping) if store else None, _ptr(q), k_ptr, v_ptr, page_stride, kv.page_size,
              kv.pages.shape[0] * kv.page_size, tokens, int(whole), int(interleaved), _code(proj.dtype),
              _ptr(error_word(proj.device)), _stream()),
           "qkv_prepare")
    return q


DECODE_CHUNK = 128
"""Keys per split of the decode attention kernel (chunks are aligned to absolute positions)."""

_scratch: dict[tuple[int, str], torch.Tensor] = {}
_zeroed: set[tuple[int, str]] = set()  # the scratch buffers that are zero between launches


def scratch(device: torch.device, name: str, numel: int, dtype: torch.dtype = torch.float32,
            zeroed: bool = False) -> torch.Tensor:
    """A reusable buffer of at least `numel` elements. Its contents are undefined unless
    `zeroed`, in which case it is zero when created and its users leave it zero."""
    key = (device.index or 0, name)
    held = _scratch.get(key)
    if held is None or held.numel() < numel or held.dtype != dtype:
        make = torch.zeros if zeroed else torch.empty
        held = _scratch[key] = make(max(numel, 1), dtype=dtype, device=device)
        if zeroed:
            _zeroed.add(key)
    return held


def _step_buffers(step: StepContext, device: torch.device, wanted: dict) -> list[torch.Tensor]:
    """Scratch buffers `name -> (elements, dtype, zeroed)` for a kernel of this step. A step whose
    workspace says `private` (a step captured into a graph, which must keep its buffers for as
    long as the graph lives) gets buffers of its own, kept in the workspace; any other step
    shares the process-wide ones. A zeroed buffer is zero when created and its users leave it zero."""
    held = step.workspace if isinstance(step.workspace, dict) else None
    private = held is not None and held.get("private", False)
    buffers = []
    for name, (numel, dtype, zeroed) in wanted.items():
        if private:
            t = held.get(name)
            if t is None or t.numel() < numel or t.dtype != dtype:
                t = held[name] = (torch.zeros if zeroed else torch.empty)(max(numel, 1), dtype=dtype, device=device)
        else:
            t = scratch(device, name, numel, dtype, zeroed)
        buffers.append(t)
    return buffers


def width_bucket(pages: int) -> int:
    """`pages` (of the longest block table of a step) rounded up to three significant bits, at
    least 8: the widths that captured decode graphs are made for, and the bound that the decode
    attention kernel's plan is made from, so that a step takes the same plan whether it runs on
    its own or from a captured graph. Rounding to powers of two would be fewer graphs, but a
    request just past 4,096 tokens would then run the grid of one of 8,192."""
    pages = max(pages, 8)
    step = 1 << max(pages.bit_length() - 3, 0)
    return -(-pages // step) * step


def decode_plan(requests: int, nkv: int, longest: int, sms: int) -> tuple[int, int]:
    """(keys per block, warps per block) of the decode attention kernel for `requests` requests
    (rounded up to a power of two, as a captured graph's batch is) of `nkv` key/value heads whose
    longest holds `longest` positions. A block of one warp walks its chunk's 32-key tiles one after
    the other, a chain of memory round trips; the GPU holds six such blocks per SM at a time, and
    measured inside whole decode steps the best plan is the one with the most blocks that still
    run in one wave: enough loads in flight to fill the memory's bandwidth, short chains, and SMs
    that all get their share. With one or two requests (at most an eighth as many (request, head)
    pairs as SMs) a block has four warps that take the chunk's tiles in turn, without a ring (a
    tile counts one and a half); at some 244 registers a thread two such blocks fit an SM (plans
    made for three ran in one and a half waves, and badly). The cost of a plan, in tile times:
    waves x (4 for a block's start and its partial result + tiles per warp), for four-warp blocks
    divided by the share of the SMs' places that they fill, + a round trip of the merge per eight
    chunks; the plan is the cheapest chunk (a multiple of 64 keys, 128 to 1024), the shorter on a
    tie. Its pick was the best or within 2 % of the best of the plans tried at 4,096 positions
    (batches 1 to 16) and at 16,000 and 32,000 (batches 1 and 2), on a GPU of 148 SMs (`sms`)."""
    pairs = (1 << max(requests - 1, 0).bit_length()) * max(nkv, 1)
    longest = max(longest, 1)
    warps, per_sm, tile = (4, 2, 1.5) if pairs * 8 <= sms else (1, 6, 1.0)
    best, best_cost = (DECODE_CHUNK, warps), None
    for chunk in range(DECODE_CHUNK, 1024 + 1, 64):
        chunks = -(-longest // chunk)
        blocks = pairs * chunks
        waves = -(-blocks // (per_sm * sms))
        filled = blocks / (min(per_sm, -(-blocks // sms)) * sms) if waves == 1 and warps == 4 else 1.0
        cost = waves * (4 + tile * -(-(chunk // 32) // warps)) / filled + -(-chunks // 8)
        if best_cost is None or cost < best_cost:
            best, best_cost = (chunk, warps), cost
    return best


def tiled_attention_supported(dtype: torch.dtype, nq: int, nkv: int, d: int) -> bool:
    """The tensor-core kernels take bfloat16, head sizes in steps of 8 up to 256 and up to
    16 query heads per key/value head; everything else runs on the generic kernel."""
    return dtype == torch.bfloat16 and d % 8 == 0 and d <= 256 and nq % nkv == 0 and nq // nkv <= 16


# The small index lists below go to the device through a ring of pinned slots that is made once:
# pinning a fresh buffer for every list cost a prefill step 0.15 ms with the GPU idle.
_STAGING_SLOTS, _STAGING_INTS = 16, 16384
_staging: dict[int, list] = {}


def _ints_to_device(values, device: torch.device) -> torch.Tensor:
    """`values` (ints, possibly nested evenly) as an int32 tensor on `device`, copied without
    blocking from a pinned slot; a slot is written again only after its last copy has finished."""
    host = torch.from_numpy(np.ascontiguousarray(values, dtype=np.int32)) if isinstance(values, np.ndarray) \
        else torch.tensor(values, dtype=torch.int32)
    if host.numel() > _STAGING_INTS:
        return host.to(device, non_blocking=True)
    index = device.index if device.index is not None else torch.cuda.current_device()
    ring = _staging.get(index)
    if ring is None:
        ring = _staging[index] = [torch.empty(_STAGING_SLOTS, _STAGING_INTS, dtype=torch.int32).pin_memory(),
                                  [None] * _STAGING_SLOTS, 0]
    slots, events, at = ring
    ring[2] = (at + 1) % _STAGING_SLOTS
    if events[at] is not None:
        events[at].synchronize()
    else:
        events[at] = torch.cuda.Event()
    pinned = slots[at, : host.numel()].view(host.shape)
    pinned.copy_(host)
    out = pinned.to(device, non_blocking=True)
    events[at].record()
    return out


def _step_list(step: StepContext, key, build, device: torch.device) -> torch.Tensor:
    """A small list of ints that a kernel of this step reads (`build(step)` makes it on the host),
    made once per step and shared by the layers. A step that is to be captured into a graph (its
    workspace says `private`) runs once uncaptured first: the list then gets a place of its own
    and its builder is kept, and the runner fills the list again before every replay of the graph
    (`fill_step_lists`): a copy made during a capture would be replayed with whatever its staging
    memory holds by then."""
    if step.workspace is None:
        step.workspace = {}
    held = step.workspace.get(key)
    if held is None:
        if step.workspace.get("private"):
            if torch.cuda.is_current_stream_capturing():
                raise KernelError(f"the list {key} of a captured step was not made before the capture")
            held = _ints_to_device(build(step), device).clone()  # a place of its own, kept with the graph
            step.workspace.setdefault("lists", {})[key] = build
        else:
            held = _ints_to_device(build(step), device)
        step.workspace[key] = held
    return held


def fill_step_lists(step: StepContext) -> None:
    """Bring the lists of a captured step up to date with the step's host-side numbers (see
    `_step_list`); each goes to the device from a pinned buffer of its own."""
    workspace = step.workspace
    pinned = workspace.setdefault("pinned", {})
    for key, build in workspace.get("lists", {}).items():
        values = np.ascontiguousarray(build(step), dtype=np.int32)
        target = workspace[key]
        if tuple(values.shape) != tuple(target.shape):
            raise KernelError(f"the list {key} changed its shape between replays of one captured step")
        host = pinned.get(key)
        if host is None:
            host = pinned[key] = torch.empty(values.shape, dtype=torch.int32).pin_memory()
        host.numpy()[...] = values
        target.copy_(host, non_blocking=True)


def _prefill_work(step: StepContext, tokens_per_block: int, device: torch.device) -> torch.Tensor:
    """(request, first token) of every block of `tokens_per_block` query tokens, the blocks
    that see the most keys first (they run longest)."""
    def build(step: StepContext) -> np.ndarray:
        items = [(s, t0) for s, n in enumerate(step.q_lens) if n > 1 for t0 in range(0, n, tokens_per_block)]
        if step.seq_lens_host:
            items.sort(key=lambda item: -(step.seq_lens_host[item[0]] - step.q_lens[item[0]] + item[1]))
        return np.asarray(items, dtype=np.int32).reshape(-1, 2)

    return _step_list(step, ("prefill_work", tokens_per_block), build, device)


PREFILL_MAX_PARTS = 16
PREFILL_MIN_PART_TILES = 12
"""The tcgen05 prefill kernel's blocks may be listed in parts (runs of a block's key tiles, merged by
the part that finishes last): at most this many parts a block, none shorter than this many tiles,
and only in steps with at most one block per SM (portions of prompts over long contexts), whose
tiles are then shared out over one and a half places per SM. Measured on B200 with the headline
model (`bench.py --only portions`, `--only mixed`), whole blocks against parts: a prompt of 8,192
tokens read in portions of 512: 68 and 53 ms, in portions of 256: 119 and 84; 32,768 tokens in
portions of 512: 586 and 328; a step of 8 decoding requests beside a 512-token portion: 6.1 and 4.9
ms. Parts of at least 4, 8, 12, 16, 24 tiles: 4.00, 3.92, 3.83, 4.23, 4.01 ms for such a step with a
256-token portion. A whole prompt has blocks enough of its own: cut, its 2,048-token attention
takes 47 us a layer against 44 (a part pays for its start, for writing its 64 KB and for the merge)."""


def prefill_places(sms: int) -> int:
    """Over how many places the tiles of a step's blocks are shared out when blocks are cut."""
    return sms + sms // 2


def prefill_blocks(step: StepContext, tokens_per_block: int, nkv: int) -> int:
    """How many blocks of query tokens (each once per key/value head) the step's prompts' portions make."""
    return sum(-(-n // tokens_per_block) for n in step.q_lens if n > 1) * nkv


def prefill_work_table(q_lens, seq_lens, tokens_per_block: int, tile: int, nkv: int, window: int, places: int,
                       capacity: int | None = None, run: int = 0) -> np.ndarray:
    """The tcgen05 prefill kernel's list, int32 [blocks, 8]: (request, first token, key/value head, first
    key tile of the part, tiles of the part (-1: all), parts + 256 * part, place of the block's first
    part in the workspace, number of the block among the split ones), the longest first: blocks are
    handed to SMs in this order as others finish, so the long ones start early and the short ones
    fill the gaps (measured: 30 % off a 4,096-token prefill against an order that keeps a head's
    blocks together).

    In a step of at most two thirds of `places` blocks, a block is cut into parts when it alone would
    run longer than a place's share of all tiles: into runs of max(that share, PREFILL_MIN_PART_TILES)
    tiles, so splitting adds at most `places` items. With `capacity` the list has
    exactly that many items, the unused ones marked with request -1 (a captured step's list keeps
    its shape from replay to replay while the contexts grow)."""
    blocks = []
    for s, n in enumerate(q_lens):
        if n <= 1:
            continue
        t0 = np.arange(0, n, tokens_per_block, dtype=np.int64)
        tiles = np.full_like(t0, -1)
        if seq_lens:
            pos0 = seq_lens[s] - n + t0
            last = pos0 + np.minimum(tokens_per_block, n - t0) - 1
            first = np.maximum(0, pos0 - window + 1) if window else np.zeros_like(t0)
            if run:  # a block's rows see no key ahead of the run of its first row
                first = np.maximum(first, pos0 - pos0 % run)
            tiles = last // tile - first // tile + 1
        # Every block of tokens once per key/value head, heads innermost.
        blocks.append(np.stack([np.repeat(tiles, nkv), np.full(t0.size * nkv, s), np.repeat(t0, nkv),
                                np.tile(np.arange(nkv), t0.size)], axis=1))
    table = np.concatenate(blocks) if blocks else np.zeros((0, 4), dtype=np.int64)
    tiles = table[:, 0]
    out = np.zeros((table.shape[0], 9), dtype=np.int64)  # column 0: the sort key
    out[:, 0], out[:, 1:4], out[:, 5], out[:, 6] = tiles, table[:, 1:4], -1, 1
    if table.shape[0] and tiles.min() > 0 and table.shape[0] * 3 <= places * 2:
        share = max(PREFILL_MIN_PART_TILES, -(-int(tiles.sum()) // places))
        wanted = np.minimum(PREFILL_MAX_PARTS, -(-tiles // share))
        per = -(-tiles // wanted)
        parts = -(-tiles // per)
        if (parts > 1).any():
            split = parts > 1
            unit = np.cumsum(split) - 1
            slot0 = np.concatenate([[0], np.cumsum(np.where(split, parts, 0))[:-1]])
            index = np.repeat(np.arange(table.shape[0]), parts)
            part = np.arange(index.size) - np.repeat(np.cumsum(parts) - parts, parts)
            rows = np.zeros((index.size, 9), dtype=np.int64)
            rows[:, 1:4] = table[index, 1:4]
            rows[:, 4] = part * per[index]
            rows[:, 5] = np.minimum(per[index], tiles[index] - rows[:, 4])
            rows[:, 6] = parts[index] + 256 * part
            rows[:, 7], rows[:, 8] = slot0[index], unit[index]
            rows[:, 0] = rows[:, 5]
            whole = ~split[index]
            rows[whole, 4], rows[whole, 5], rows[whole, 6], rows[whole, 0] = 0, -1, 1, tiles[index][whole]
            out = rows
    order = np.argsort(-out[:, 0], kind="stable")
    out = out[order, 1:].astype(np.int32)
    if capacity is not None:
        if out.shape[0] > capacity:
            raise KernelError(f"the prefill kernel's list has {out.shape[0]} items, its place holds {capacity}")
        padded = np.full((capacity, 8), -1, dtype=np.int32)
        padded[: out.shape[0]] = out
        out = padded
    return out


WIDE_MIN_TOKENS = 512
WIDE_MIN_WINDOW = 1024


def wide_prefill_pays(q_lens, seq_lens, tokens_per_block: int, nkv: int, window: int, sms: int) -> bool:
    """Which of the two tcgen05 prefill kernels a step's prompts take: True for the one that gives a
    block an SM of its own (attention_tcgen05_wide.cu), False for the one that runs two blocks to an
    SM and cuts long blocks into parts (attention_tcgen05.cu).

    Measured on a B200 (16 query and 8 key/value heads of 128, with the gate; us, wide against two to
    an SM; a prompt of n tokens makes n / 64 blocks per key/value head): one whole prompt of 512 / 1,024
    / 2,048 / 2,304 tokens 17 / 19 / 37 / 42 against 22 / 24 / 44 / 52 (few blocks, each a long chain of
    tiles, which a block alone on its SM walks at 1.16 us for 128 keys against 1.06 us for 64), of
    2,560 / 2,816 / 3,072: 53 / 61 / 68 against 57 / 60 / 65, of 4,096 / 8,192: 101 / 323 against 88 / 290
    (a block's 7 us of start and epilogue overlap nothing when it has its SM alone); 2 prompts of 768
    or of 1,024, 4 of 512: even; 2 of 1,536, 3 of 1,024 (384 blocks): 48 / 40 against 39 / 31; 8
    portions of 256 over 1,024: 36 against 31; 512 over 8,192 cut into parts: 75 against 57. So:
    prompts from their first token, each of at least WIDE_MIN_TOKENS tokens, at most two blocks to an
    SM, and no window shorter than WIDE_MIN_WINDOW. The answer depends on the step's lengths and on
    whether its prompts start at zero, both of which a captured step's key holds."""
    prompts = [(n, held) for n, held in zip(q_lens, seq_lens or ()) if n > 1]
    if not prompts or any(held != n or n < WIDE_MIN_TOKENS for n, held in prompts):
        return False
    blocks = sum(-(-n // tokens_per_block) for n, _ in prompts) * nkv
    return blocks <= 2 * sms and (not window or window >= WIDE_MIN_WINDOW)


def _prefill_work_flat(step: StepContext, tokens_per_block: int, tile: int, nkv: int, window: int,
                       device: torch.device, places: int, run: int = 0) -> torch.Tensor:
    """The list of `prefill_work_table` for this step, made once and shared by the layers of equal window and run."""
    capacity = prefill_blocks(step, tokens_per_block, nkv) + places if (step.workspace or {}).get("private") else None
    build = lambda st: prefill_work_table(st.q_lens, st.seq_lens_host, tokens_per_block, tile, nkv, window, places, capacity,
                                          run)
    return _step_list(step, ("prefill_work_flat", tokens_per_block, tile, nkv, window, places, run), build, device)


def single_token_longest(step: StepContext) -> int:
    """The longest of the requests that bring one token to a mixed step (they take the decode kernel)."""
    return max((n for q, n in zip(step.q_lens, step.seq_lens_host) if q == 1), default=0)


def _single_token_requests(step: StepContext, device: torch.device) -> tuple[torch.Tensor | None, int]:
    """Indices of the requests that bring one token to a mixed step, and the longest of them."""
    ids = [s for s, n in enumerate(step.q_lens) if n == 1]
    if not ids:
        return None, 0
    return _step_list(step, "single_token_requests", lambda _: np.asarray(ids, dtype=np.int32), device), \
        single_token_longest(step)


def tcgen05_attention_supported(dtype: torch.dtype, nq: int, nkv: int, d: int, page_size: int) -> bool:
    """The tcgen05 prefill kernel takes bfloat16, head sizes 64 and 128, pages of a multiple
    of 16 tokens and up to 16 query heads per key/value head."""
    return (dtype == torch.bfloat16 and d in (64, 128) and page_size % 16 == 0 and nq % nkv == 0
            and nq // nkv <= 16)


@dataclass
class Projection:
    """A decode step's projected rows, for the decode attention kernel to normalise, rotate and
    store by itself (what `qk_norm_rope_store` would do in a kernel of its own)."""
    rows: torch.Tensor  # [tokens, stride]
    q_col: int
    k_col: int
    v_col: int
    nq: int
    d: int
    eps: float | None
    inv_freq: torch.Tensor | None


def decode_fusable(proj: torch.Tensor, nq: int, nkv: int, d: int, inv_freq: torch.Tensor | None,
                   kv: KVView, step: StepContext) -> bool:
    """Whether the decode attention kernel can take the projected rows as they are: a step of
    single tokens, bfloat16, a head size that is a multiple of 32, rotated whole or not at all,
    and a cache entry that this layer writes."""
    return (step.decode_only and proj.is_cuda and kv.writes and d % 32 == 0
            and (inv_freq is None or 2 * inv_freq.shape[0] == d) and proj.shape[1] % 2 == 0
            and tiled_attention_supported(proj.dtype, nq, nkv, d))


def paged_attention(q: torch.Tensor | None, kv: KVView, step: StepContext, scale: float,
                    gate: torch.Tensor | None = None, gate_col: int = 0,
                    projection: Projection | None = None, wide: bool | None = None,
                    sink: torch.Tensor | None = None, window: int | None = -1,
                    keep_first: int | None = None, chunk: int | None = None,
                    softcap: float | None = None) -> torch.Tensor:
    """Causal (windowed) attention of this step's queries over the paged cache, the
    output multiplied by sigmoid(gate) when `gate` (the projected rows; the gate's
    columns start at `gate_col`) is given.  -> [tokens, nq * dv]

    `sink` (float32 [nq]) adds exp(sink[head]) to every row's denominator. A cache whose spec names
    `keep_first` keeps that many first positions visible behind the window; `window` and `keep_first`,
    when given, are the mixer's own and replace the cache's (a mixer that reads another's cache may
    see less of it than is kept). Sink and kept positions are taken by the generic kernel, by the
    mma.sync kernels and by the tcgen05 prefill kernel that runs two blocks to an SM (every block is
    then listed whole), not by the one that gives a block its SM; values of another width than the
    keys run on the generic kernel.

    `chunk` n: a query sees only the keys of its own run of n positions (runs counted from the request's
    position 0, wherever a prompt was cut); `softcap` c: a scaled score s becomes c tanh(s / c) ahead of
    the softmax. Both are taken by the generic kernel, by the mma.sync kernels and by the tcgen05 prefill
    kernel that runs two blocks to an SM.

    With `projection` (only where `decode_fusable` holds) q is not given: the kernel makes the
    queries and the new keys and values from the projected rows, and writes the latter to the cache.

    bfloat16 with a supported head size runs on the tensor-core kernels: the split-key
    decode kernel when every request brings one token; otherwise the tcgen05 prefill kernel
    (head sizes 64 and 128, pages of a multiple of 16) or the mma.sync prefill kernel. Other
    cases (the 32-bit path among them) run on the generic kernel."""
    if projection is not None:
        tokens, nq, d = projection.rows.shape[0], projection.nq, projection.d
        q = projection.rows  # for its dtype and device only
    else:
        tokens, nq, d = q.shape
    k_ptr, v_ptr, page_stride, nkv, _, dv = kv_layout(kv)
    if window != -1 and (window or 0) != (kv.window or 0):
        kv = dataclasses.replace(kv, window=window)
    keep = kv.keep_first if keep_first is None else keep_first
    if not kv.window:
        keep = 0
    out = torch.empty(tokens, nq * dv, dtype=q.dtype, device=q.device)
    gate_ptr = None if gate is None else gate.data_ptr() + gate_col * gate.element_size()
    gate_stride = 0 if gate is None else gate.shape[1]
    err = _ptr(error_word(q.device))
    max_pages, num_pages = kv.block_table.shape[1], kv.pages.shape[0]
    run, softcap = int(chunk or 0), float(softcap or 0.0)
    if run and keep:
        raise KernelError("a mask of runs keeps no first positions")
    if dv != d or not tiled_attention_supported(q.dtype, nq, nkv, d):
        if projection is not None:
            raise KernelError("the generic attention kernel takes queries, not projected rows")
        fn = _function("attention_generic", "omnia_paged_attention_generic",
                       [c_void_p, c_void_p, c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                        c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                        c_int, c_float, c_int, c_float, c_int, c_void_p, c_void_p])
        _check(fn(_ptr(q), k_ptr, v_ptr, page_stride, _ptr(kv.block_table), _ptr(step.cu_seqlens),
                  _ptr(step.positions), gate_ptr, gate_stride, _ptr(out), _ptr(sink), tokens, step.num_seqs, max_pages,
                  num_pages, nq, nkv, d, dv, kv.page_size, kv.window or 0, keep, scale, run, softcap,
                  _code(q.dtype), err, _stream()), "paged_attention")
        return out
    defines = {"HEAD_DIM": d, "GROUP": nq // nkv}
    # Requests that bring a single token take the split-key decode kernel, in a decode-only step
    # (all of them, no index list: the shape a captured graph replays) and in a mixed step alike.
    single, longest = (None, step.max_seq_len) if step.decode_only else _single_token_requests(step, q.device)
    if step.decode_only or single is not None:
        count = step.num_seqs if step.decode_only else single.shape[0]
        longest = width_bucket(-(-longest // kv.page_size)) * kv.page_size
        chunk, warps = decode_plan(count, nkv, longest, sm_count(q.device))
        max_chunks = -(-longest // chunk)
        part_o, part_ml, tickets = _step_buffers(step, q.device, {
            "attention_part_o": (count * nq * max_chunks * d, torch.float32, False),
            "attention_part_ml": (count * nq * max_chunks * 2, torch.float32, False),
            "attention_tickets": (count * nkv, torch.int32, True)})
        fn = _function("attention_tc", "omnia_attention_decode_tc",
                       [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p,
                        c_void_p, c_int, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
                        c_float, c_int, c_void_p, c_int, c_int, c_int, c_int, c_float, c_void_p, c_void_p,
                        c_int, c_int, c_void_p, c_int, c_float, c_void_p, c_void_p], defines)
        p = projection
        fused = (None, 0, 0, 0, 0, -1.0, None, None) if p is None else (
            _ptr(p.rows), p.rows.shape[1], p.q_col, p.k_col, p.v_col, -1.0 if p.eps is None else p.eps,
            _ptr(p.inv_freq), _ptr(kv.slot_mapping))
        _check(fn(None if p is not None else _ptr(q), _ptr(kv.pages), _ptr(kv.block_table), _ptr(step.cu_seqlens),
                  _ptr(step.seq_lens), _ptr(single), count, _ptr(part_o), _ptr(part_ml), _ptr(tickets), chunk,
                  max_chunks, gate_ptr, gate_stride, _ptr(out), max_pages, num_pages, nq, nkv, kv.page_size,
                  kv.window or 0, scale, warps, *fused, 1, keep, _ptr(sink), run, softcap, err, _stream()),
               "attention_decode")
        if step.decode_only or all(n == 1 for n in step.q_lens):
            return out
    if tcgen05_attention_supported(q.dtype, nq, nkv, d, kv.page_size):
        per_block = 128 // (nq // nkv)
        sms = sm_count(q.device)
        plain = sink is None and not keep  # a sink or kept first positions: the two-to-an-SM kernel, every block whole
        narrow = bool(run or softcap)  # runs and capped scores: the two-to-an-SM kernel, blocks cut as ever
        if wide is None:
            wide = plain and not narrow and wide_prefill_pays(step.q_lens, step.seq_lens_host, per_block, nkv,
                                                              kv.window or 0, sms)
        elif wide and (not plain or narrow):
            raise KernelError("the kernel that gives a block its SM takes no sink, kept first positions, runs or cap")
        if wide:
            # Every block whole (no places to share tiles over), an SM to a block.
            work = _prefill_work_flat(step, per_block, 64, nkv, kv.window or 0, q.device, 0)
            fn = _function("attention_tcgen05_wide", "omnia_attention_prefill_tcgen05_wide",
                           [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int,
                            c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_void_p, c_void_p], defines)
            _check(fn(_ptr(q), tokens, _ptr(kv.pages), _ptr(kv.block_table), _ptr(step.cu_seqlens), _ptr(step.seq_lens),
                      _ptr(work), work.shape[0], gate_ptr, gate_stride, _ptr(out), max_pages, num_pages, nq, nkv,
                      kv.page_size, kv.window or 0, scale, err, _stream()), "attention_prefill_tcgen05_wide")
            return out
        work = _prefill_work_flat(step, per_block, 64, nkv, kv.window or 0, q.device, prefill_places(sms) if plain else 0,
                                  run)
        # Room for the parts of blocks that are cut (at most one more item per block the device runs at
        # a time) and a ticket per block; the sizes do not depend on the contexts' lengths.
        part_floats = _function("attention_tcgen05", "omnia_attention_tcgen05_part_floats", [], defines)()
        base = prefill_blocks(step, per_block, nkv)
        partial, tickets = _step_buffers(step, q.device, {
            "prefill_parts": ((base + prefill_places(sms)) * part_floats, torch.float32, False),
            "prefill_tickets": (base, torch.int32, True)})
        fn = _function("attention_tcgen05", "omnia_attention_prefill_tcgen05",
                       [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int,
                        c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_void_p,
                        c_int, c_float, c_void_p, c_void_p], defines)
        _check(fn(_ptr(q), tokens, _ptr(kv.pages), _ptr(kv.block_table), _ptr(step.cu_seqlens), _ptr(step.seq_lens),
                  _ptr(work), work.shape[0], gate_ptr, gate_stride, _ptr(out), _ptr(partial), _ptr(tickets), max_pages,
                  num_pages, nq, nkv, kv.page_size, kv.window or 0, scale, keep, _ptr(sink), run, softcap, err, _stream()),
               "attention_prefill_tcgen05")
        return out
    tokens_per_block = 64 // (nq // nkv)
    work = _prefill_work(step, tokens_per_block, q.device)
    fn = _function("attention_tc", "omnia_attention_prefill_tc",
                   [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p,
                    c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_void_p, c_int, c_float, c_void_p,
                    c_void_p], defines)
    _check(fn(_ptr(q), _ptr(kv.pages), _ptr(kv.block_table), _ptr(step.cu_seqlens), _ptr(step.seq_lens), _ptr(work),
              work.shape[0], gate_ptr, gate_stride, _ptr(out), max_pages, num_pages, nq, nkv, kv.page_size,
              kv.window or 0, scale, keep, _ptr(sink), run, softcap, err, _stream()), "attention_prefill")
    return out


def swiglu(gu: torch.Tensor) -> torch.Tensor:
    """act = silu(gu[:, :inner]) * gu[:, inner:]"""
    rows, two_inner = gu.shape
    inner = two_inner // 2
    act = torch.empty(rows, inner, dtype=gu.dtype, device=gu.device)
    fn = _function("elementwise", "omnia_swiglu", [c_void_p, c_void_p, c_int, c_int, c_int, c_void_p])
    _check(fn(_ptr(gu), _ptr(act), rows, inner, _code(gu.dtype), _stream()), "swiglu")
    return act


def clamped_glu(gu: torch.Tensor, alpha: float, limit: float) -> torch.Tensor:
    """g = min(gu[:, :inner], limit), u = clamp(gu[:, inner:], -limit, limit); act = g sigmoid(alpha g) (u + 1)."""
    rows, two_inner = gu.shape
    inner = two_inner // 2
    act = torch.empty(rows, inner, dtype=gu.dtype, device=gu.device)
    fn = _function("elementwise", "omnia_clamped_glu", [c_void_p, c_void_p, c_int, c_int, c_float, c_float, c_int, c_void_p])
    _check(fn(_ptr(gu), _ptr(act), rows, inner, alpha, limit, _code(gu.dtype), _stream()), "clamped_glu")
    return act


def softcap(z: torch.Tensor, multiplier: float, cap: float | None) -> torch.Tensor:
    """float32 logits = cap * tanh(z * multiplier / cap); no cap when `cap` is None."""
    out = torch.empty(z.shape, dtype=torch.float32, device=z.device)
    fn = _function("elementwise", "omnia_softcap", [c_void_p, c_void_p, c_longlong, c_float, c_float, c_int, c_void_p])
    _check(fn(_ptr(z), _ptr(out), z.numel(), multiplier, cap or 0.0, _code(z.dtype), _stream()), "softcap")
    return out


def gather_rows(src: torch.Tensor, rows: torch.Tensor) -> torch.Tensor:
    """out[r] = src[rows[r]]"""
    count, width = rows.shape[0], src.shape[1]
    out = torch.empty(count, width, dtype=src.dtype, device=src.device)
    fn = _function("elementwise", "omnia_gather_rows", [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p])
    _check(fn(_ptr(src), _ptr(rows), _ptr(out), count, width, _code(src.dtype), _stream()), "gather_rows")
    return out


SKINNY_ROWS = 16
"""Up to this many activation rows, bfloat16 products run on the weight-streaming kernel."""

FUSED_GATE_ROWS = 320
FUSED_CAP_ROWS = 129
"""From these many rows on, the products that have an epilogue fused into them (gate‖up with SwiGLU;
the head with its soft cap) run on this package's tcgen05 kernels. Measured on B200 inside replayed
graphs (weights of 8 to 50 MB, fresh for every launch): gate‖up with SwiGLU takes 46.7 us at 1,024
rows, 87.5 at 2,048 and 305 at 8,192, against 58.7, 112 and 408 for the vendor library's product
followed by the SwiGLU kernel; at 384 / 512 / 640 / 768 / 896 rows 24.3 / 31.0 / 34.6 / 35.0 / 46.3
against 26.7 / 33.8 / 41.5 / 43.0 / 55.5 (the kernel with one SM or two to a tile, whichever runs fewer
waves: `_pair_pays`); at 264 rows the library's pair is the faster one (23.3 against 24.1 us).

A product with nothing fused into it is the vendor library's above the streaming kernel's rows, as the
reference's is MLX's. The tcgen05 kernels take the same products (`_gemm_tcgen05`, tested), but the
library is ahead at every size measured: by 3 to 10 % at 2,048 to 4,096 rows (38.5 against 39.6 us
for 2,048 x 6,144 x 2,048), by 1.3 to 2.8 times between 129 and 1,024 rows, where 128 x 256 tiles
are too few for the SMs (12.1 against 33.8 us for 264 x 2,048 x 6,144), and by 10 to 28 % at 8,192.
Two kernels of this package's own for the rows in between were built, right and deterministic, and
not kept: the weights as the 128-row operand of tcgen05.mma with the few activation rows as its
columns (a tcgen05.mma with M = 128 occupies the tensor core for some 80 ns however few columns it
has, so the weights stream at half the rate of 256-column tiles), and the k range of a 128 x 256 tile
cut over a thread-block cluster (the exchange of partial sums, 128 KB a block, costs what the cut
saves: 10.6 to 32 us against the library's 8 to 12)."""

PENDING_MAX_ROWS = 8
PENDING_MAX_WIDTH = 2048
"""The most rows and the widest residual stream whose pending step the weight-streaming kernel runs itself."""

def _skinny(a: torch.Tensor, weight: torch.Tensor) -> bool:
    return (a.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and 0 < a.shape[0] <= SKINNY_ROWS
            and a.shape[1] % 8 == 0 and a.is_cuda and a.is_contiguous() and weight.is_contiguous()
            and a.data_ptr() % 16 == 0 and weight.data_ptr() % 16 == 0)


def _tensor_core(a: torch.Tensor, weight: torch.Tensor, rows: int) -> bool:
    """Whether a product with a fused epilogue runs on the tcgen05 kernels (from `rows` rows on)."""
    return (a.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and a.is_cuda
            and a.shape[0] >= rows and a.shape[1] % 8 == 0 and a.is_contiguous()
            and weight.is_contiguous())


def _pair_pays(rows: int, n: int, k: int, epilogue: int, sms: int) -> bool:
    """Whether the two-SM kernel is the faster one: it brings in a third less per step of k, but
    has half as many (twice as large) tiles to hand out and a longer start. Measured on a GPU of
    148 SMs it wins by 4 to 13 % where a pair of SMs gets at least 64 steps of k of a 256 x 256
    tile to do (2,048 rows of 2,048 columns times 6,144 or more; 8,192 rows: all), and loses where
    the work is less (2,048 x 2,048 x 2,048; 512 rows)."""
    if rows < 256:
        return False
    if epilogue == 1:
        # gate|up with SwiGLU: tiles of 128 output columns, 128 rows to an SM or 256 to a pair. What
        # decides is how many waves of tiles each kernel runs (measured, 12,288 weight rows of 2,048:
        # some 10 us and 14 a wave for one SM, 8 and 13 a wave for a pair; 264 / 512 / 768 / 896 rows:
        # 24 / 38 / 38 / 51 us against 30 / 31 / 35 / 46).
        tiles = -(-(n // 2) // 128)
        one = -(-(-(-rows // 128) * tiles) // sms)
        two = -(-(-(-rows // 256) * tiles) // (sms // 2))
        return 8 + 13 * two < 10 + 14 * one
    tiles = -(-rows // 256) * -(-n // 256)
    return tiles * -(-k // 64) >= 64 * (sms // 2)


def _gemm_tcgen05(a: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, epilogue: int, multiplier: float = 1.0,
                  cap: float = 0.0, pair: bool | None = None) -> torch.Tensor:
    """The product on one of the two tcgen05 kernels: two SMs to a tile where that pays (`pair` None),
    or the one the caller names."""
    if pair is None:
        pair = _pair_pays(a.shape[0], weight.shape[0], a.shape[1], epilogue, sm_count(a.device))
    library, name = ("gemm_tcgen05_pair", "omnia_gemm_tcgen05_pair") if pair else ("gemm_tcgen05", "omnia_gemm_tcgen05")
    fn = _function(library, name,
                   [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_float, c_float, c_void_p, c_void_p])
    _check(fn(_ptr(a), _ptr(weight), _ptr(out), a.shape[0], weight.shape[0], a.shape[1], epilogue, multiplier, cap,
              _ptr(error_word(a.device)), _stream()), library)
    return out


def begin_pass(step: StepContext) -> None:
    """A pass over the model's layers begins: what kernels keep for the length of one pass (tables
    made from the step's positions, shared by the layers) is made afresh. A captured step is the
    same object from replay to replay, and its capture must hold the kernels that make them."""
    if isinstance(step.workspace, dict):
        step.workspace.pop("pass", None)


def rope_angles(step: StepContext, inv_freq: torch.Tensor) -> torch.Tensor:
    """(cos, sin)(position * inv_freq) for every token of the step, float32 [len(inv_freq), tokens, 2],
    made once per pass and per table of frequencies (layers of one base share it)."""
    if step.workspace is None:
        step.workspace = {}
    made = step.workspace.setdefault("pass", {})
    key = ("rope_angles", inv_freq.data_ptr())
    table = made.get(key)
    if table is None:
        half = inv_freq.shape[0]
        (table,) = _step_buffers(step, inv_freq.device,
                                 {f"rope_angles_{inv_freq.data_ptr()}": (step.num_tokens * half * 2, torch.float32, False)})
        fn = _function("elementwise", "omnia_rope_angles", [c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p])
        _check(fn(_ptr(step.positions), _ptr(inv_freq), half, step.num_tokens, _ptr(table), _stream()), "rope_angles")
        made[key] = table
    return table


FUSED_QKV_ROWS = 1280
"""From how many rows on the attention input projection runs on the two-SM tcgen05 kernel with the
head norms, the rotation and the cache write in its epilogue, instead of the library's product and
the kernel that reads its result back. B200, rows x 2,048 -> 6,144, us for the two against the one
(without the 3 us of the angles' table, which a pass makes once for all its layers): 768 rows 22.7
against 23.2, 1,024: 29.4 against 29.7, 1,280: 34.8 against 31.2, 1,536: 37.2 against 31.7, 2,048:
50.7 against 42.9, 4,096: 94.0 against 80.8, 8,192: 182.7 against 154.8 (the bare products at
2,048 rows: 38.8 us for this kernel, 37.3 for the library's)."""


def linear_qkv(x, weight: torch.Tensor, q_col: int, k_col: int, v_col: int, nq: int, nkv: int, d: int,
               eps: float | None, inv_freq: torch.Tensor | None, step: StepContext,
               kv: KVView | None) -> tuple[torch.Tensor, torch.Tensor] | None:
    """x @ weight.T for weight = [q | (gate) | k | v] rows, with `qk_norm_rope_store` done in the
    product's epilogue: -> (the projected rows, of which only the columns that are neither q, k nor
    v are written; q as [tokens, nq, d]), k and v in the cache pages. None where this does not
    apply (few rows, another dtype, a head size other than 64 or 128, a rotation of part of the
    head): the caller then takes the product and `qk_norm_rope_store` one after the other."""
    store = kv is not None and kv.writes
    if not (isinstance(x, torch.Tensor) and _tensor_core(x, weight, FUSED_QKV_ROWS) and d in (64, 128)
            and (inv_freq is None or 2 * inv_freq.shape[0] == d) and weight.shape[0] % d == 0
            and q_col % d == 0 and (not store or (k_col % d == 0 and v_col % d == 0 and kv.pages.dtype == torch.bfloat16))):
        return None
    rows, n = x.shape[0], weight.shape[0]
    proj = torch.empty(rows, n, dtype=x.dtype, device=x.device)
    q = torch.empty(rows, nq, d, dtype=x.dtype, device=x.device)
    angles = None if inv_freq is None else rope_angles(step, inv_freq)
    fn = _function("gemm_tcgen05_pair", "omnia_gemm_tcgen05_pair_qkv",
                   [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float,
                    c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_longlong, c_void_p, c_void_p])
    _check(fn(_ptr(x), _ptr(weight), _ptr(proj), rows, n, x.shape[1], d, q_col, k_col if store else 0, v_col if store else 0,
              nq, nkv if store else 0, -1.0 if eps is None else eps, _ptr(angles), _ptr(kv.slot_mapping) if store else None,
              _ptr(q), _ptr(kv.pages) if store else None, kv.page_size if store else 1,
              kv.pages.shape[0] * kv.page_size if store else 0, _ptr(error_word(x.device)), _stream()), "gemm_tcgen05_pair_qkv")
    return proj, q


def _library_mm(a: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    if a.dtype == torch.float32 and (torch.backends.cuda.matmul.allow_tf32
                                      or torch.get_float32_matmul_precision() != "highest"):
        raise KernelError("the 32-bit path needs true float32 matrix products; TF32 is switched on")
    return torch.mm(a, weight.t())


def _gemv_stream(a: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, epilogue: int, multiplier: float = 1.0,
                 cap: float = 0.0) -> torch.Tensor:
    """The product of up to 16 rows on the weight-streaming kernel (epilogue 0 store, 1 SwiGLU, 2 soft cap)."""
    fn = _function("gemv_stream", "omnia_gemv_stream",
                   [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_float, c_float, c_void_p, c_void_p])
    _check(fn(_ptr(a), _ptr(weight), _ptr(out), a.shape[0], weight.shape[0], a.shape[1], epilogue, multiplier, cap,
              _ptr(error_word(a.device)), _stream()), "gemv_stream")
    return out


@dataclass
class PendingStep:
    """A residual step that has not run yet: x_new = x + norm_b(branch), h = norm_o(x_new). The
    product that takes h (`linear`, `linear_swiglu`) runs it in its own kernel where it can, and
    anything else settles it first with `settle`. Either way `x_new` then holds the new residual
    (a buffer of its own when a product ran the step, since a kernel whose blocks all read x
    cannot update it in place; x itself otherwise)."""

    x: torch.Tensor
    branch: torch.Tensor
    branch_weight: torch.Tensor | None
    branch_eps: float | None
    out_weight: torch.Tensor | None
    out_eps: float
    x_new: torch.Tensor | None = None
    h: torch.Tensor | None = None


def pending_supported(x: torch.Tensor, branch: torch.Tensor) -> bool:
    """Whether a product of this step's rows could run the residual step itself."""
    return (x.is_cuda and branch.dtype == torch.bfloat16 and 0 < x.shape[0] <= PENDING_MAX_ROWS
            and x.shape[1] % 8 == 0 and x.shape[1] <= PENDING_MAX_WIDTH and x.is_contiguous()
            and branch.is_contiguous())


def settle(h):
    """The activations of `h`; a pending step is run now, by the kernel of its own."""
    if not isinstance(h, PendingStep):
        return h
    if h.x_new is None:
        h.h = add_rmsnorm(h.x, h.branch, h.branch_weight, h.branch_eps, h.out_weight, h.out_eps)
        h.x_new = h.x
    if h.h is None:
        raise RuntimeError("a pending residual step was already consumed by a product; its activations were not kept")
    return h.h


def residual_after(h, x: torch.Tensor) -> torch.Tensor:
    """The residual stream after whatever took `h` has run: `x` itself, or the new residual of a
    pending step (settled now if nothing took it)."""
    if not isinstance(h, PendingStep):
        return x
    if h.x_new is None:
        settle(h)
    return h.x_new


def _pending_product(step: PendingStep, weight: torch.Tensor, epilogue: int) -> torch.Tensor | None:
    """The product with the pending step in front, or None where the kernel does not take it."""
    if step.x_new is not None or not (weight.dtype == torch.bfloat16 and weight.shape[1] == step.x.shape[1]
                                      and weight.data_ptr() % 16 == 0 and weight.is_contiguous()
                                      and pending_supported(step.x, step.branch)):
        return None
    rows, n = step.x.shape[0], weight.shape[0]
    out = torch.empty(rows, n // 2 if epilogue == 1 else n, dtype=torch.bfloat16, device=step.x.device)
    x_new = torch.empty_like(step.x)
    fn = _function("gemv_stream", "omnia_gemv_stream_pending",
                   [c_void_p, c_void_p, c_void_p, c_void_p, c_float, c_int, c_void_p, c_float, c_void_p, c_void_p,
                    c_int, c_int, c_int, c_int, c_void_p, c_void_p])
    _check(fn(_ptr(step.x), _ptr(x_new), _ptr(step.branch), _ptr(step.branch_weight), step.branch_eps or 0.0,
              int(step.branch_eps is not None), _ptr(step.out_weight), step.out_eps, _ptr(weight), _ptr(out), rows, n,
              weight.shape[1], epilogue, _ptr(error_word(step.x.device)), _stream()), "gemv_stream_pending")
    step.x_new = x_new
    return out


def linear(a, weight: torch.Tensor) -> torch.Tensor:
    """a [rows, k] times weight [n, k] transposed -> [rows, n], float32 accumulation.
    A few bfloat16 rows (a decode step) run on this package's weight-streaming kernel, with the
    pending residual step fused in front. Otherwise the matrix product is the vendor library's (as
    the reference's is MLX's); on the 32-bit path it runs without any reduced-precision mode.
    `a` may be a PendingStep."""
    if isinstance(a, PendingStep):
        out = _pending_product(a, weight, 0)
        if out is not None:
            return out
        a = settle(a)
    if _skinny(a, weight):
        return _gemv_stream(a, weight, torch.empty(a.shape[0], weight.shape[0], dtype=a.dtype, device=a.device), 0)
    return _library_mm(a, weight)


def linear_add(a: torch.Tensor, weight: torch.Tensor, alpha: float, other: torch.Tensor, beta: float) -> torch.Tensor:
    """alpha * (a @ weight^T) + beta * other -> [rows, n], the sum taken on the product's float32
    accumulators and rounded once: the vendor library's product with both constants in its epilogue. A
    few bfloat16 rows run on the weight-streaming kernel and meet `other` in a pass of their own."""
    if _skinny(a, weight):
        return scaled_sum(linear(a, weight), alpha, other, beta)
    if a.dtype == torch.float32 and (torch.backends.cuda.matmul.allow_tf32
                                      or torch.get_float32_matmul_precision() != "highest"):
        raise KernelError("the 32-bit path needs true float32 matrix products; TF32 is switched on")
    return torch.addmm(other, a, weight.t(), beta=beta, alpha=alpha)


def linear_swiglu(a, gate_up: torch.Tensor) -> torch.Tensor:
    """silu(a @ gate^T) * (a @ up^T) with gate_up = [gate rows | up rows] -> [rows, inner].
    `a` may be a PendingStep."""
    if isinstance(a, PendingStep):
        out = _pending_product(a, gate_up, 1)
        if out is not None:
            return out
        a = settle(a)
    if _skinny(a, gate_up):
        return _gemv_stream(a, gate_up, torch.empty(a.shape[0], gate_up.shape[0] // 2, dtype=a.dtype, device=a.device), 1)
    if _tensor_core(a, gate_up, FUSED_GATE_ROWS):
        return _gemm_tcgen05(a, gate_up, torch.empty(a.shape[0], gate_up.shape[0] // 2, dtype=a.dtype, device=a.device), 1)
    return swiglu(_library_mm(a, gate_up))


def linear_clamped_glu(a: torch.Tensor, gate_up: torch.Tensor, alpha: float, limit: float) -> torch.Tensor:
    """g = min(a @ gate^T, limit), u = clamp(a @ up^T, -limit, limit); g sigmoid(alpha g) (u + 1), with
    gate_up = [gate rows | up rows] -> [rows, inner]. The unit sits in the product's epilogue where
    SwiGLU does: the weight-streaming kernel up to 16 rows, the tcgen05 kernels from FUSED_GATE_ROWS
    on; in between, and on the 32-bit path, the library's product and the unit's own kernel."""
    if limit <= 0:
        raise KernelError(f"the clamped gated unit needs a positive limit, got {limit}")
    if _skinny(a, gate_up):
        out = torch.empty(a.shape[0], gate_up.shape[0] // 2, dtype=a.dtype, device=a.device)
        return _gemv_stream(a, gate_up, out, 1, alpha, limit)
    if _tensor_core(a, gate_up, FUSED_GATE_ROWS):
        out = torch.empty(a.shape[0], gate_up.shape[0] // 2, dtype=a.dtype, device=a.device)
        return _gemm_tcgen05(a, gate_up, out, 1, alpha, limit)
    return clamped_glu(_library_mm(a, gate_up), alpha, limit)


def linear_relu_glu(a, gate_up: torch.Tensor) -> torch.Tensor:
    """relu(a @ gate^T) * (a @ up^T) with gate_up = [gate rows | up rows] -> [rows, inner]. The unit sits
    where SwiGLU does (the gated epilogues' third form, selected by a negative limit): the
    weight-streaming kernel up to 16 rows, the tcgen05 kernels from FUSED_GATE_ROWS on; in between,
    and on the 32-bit path, the library's product and the unit's own kernel. `a` may be a PendingStep."""
    a = settle(a)
    if _skinny(a, gate_up):
        out = torch.empty(a.shape[0], gate_up.shape[0] // 2, dtype=a.dtype, device=a.device)
        return _gemv_stream(a, gate_up, out, 1, 1.0, -1.0)
    if _tensor_core(a, gate_up, FUSED_GATE_ROWS):
        out = torch.empty(a.shape[0], gate_up.shape[0] // 2, dtype=a.dtype, device=a.device)
        return _gemm_tcgen05(a, gate_up, out, 1, 1.0, -1.0)
    gu = _library_mm(a, gate_up)
    rows, inner = gu.shape[0], gu.shape[1] // 2
    act = torch.empty(rows, inner, dtype=gu.dtype, device=gu.device)
    fn = _function("elementwise", "omnia_clamped_glu", [c_void_p, c_void_p, c_int, c_int, c_float, c_float, c_int, c_void_p])
    _check(fn(_ptr(gu), _ptr(act), rows, inner, 1.0, -1.0, _code(gu.dtype), _stream()), "relu_glu")
    return act


def linear_softcap(a: torch.Tensor, weight: torch.Tensor, multiplier: float, cap: float | None) -> torch.Tensor:
    """float32 logits = cap * tanh((a @ weight^T) * multiplier / cap) -> [rows, n]."""
    if _skinny(a, weight):
        out = torch.empty(a.shape[0], weight.shape[0], dtype=torch.float32, device=a.device)
        return _gemv_stream(a, weight, out, 2, multiplier, cap or 0.0)
    if _tensor_core(a, weight, FUSED_CAP_ROWS):
        out = torch.empty(a.shape[0], weight.shape[0], dtype=torch.float32, device=a.device)
        return _gemm_tcgen05(a, weight, out, 2, multiplier, cap or 0.0)
    return softcap(_library_mm(a, weight), multiplier, cap)


def argmax(logits: torch.Tensor) -> torch.Tensor:
    """The first largest entry of each row of float32 `logits` [rows, vocab]. -> int32 [rows]"""
    rows, vocab = logits.shape
    out = torch.empty(rows, dtype=torch.int32, device=logits.device)
    part_v = scratch(logits.device, "argmax_v", rows * 32)
    part_i = scratch(logits.device, "argmax_i", rows * 32, torch.int32)
    fn = _function("sampling", "omnia_argmax", [c_void_p, c_longlong, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p])
    _check(fn(_ptr(logits), logits.stride(0), rows, vocab, _ptr(part_v), _ptr(part_i), _ptr(out), _stream()), "argmax")
    return out


def sample(logits: torch.Tensor, temperature: torch.Tensor, top_k: torch.Tensor, top_p: torch.Tensor,
           min_p: torch.Tensor, seeds: torch.Tensor, draws: torch.Tensor, penalty: torch.Tensor | None = None,
           history: torch.Tensor | None = None) -> torch.Tensor:
    """One token per row of float32 logits [rows, vocab] (the rows are modified when a
    repetition penalty applies). Per-row parameters: temperature (0 = greedy), top_k
    (0 = off), top_p (1 = off), min_p (0 = off), seed and draw index (int64). -> int32 [rows]"""
    rows, vocab = logits.shape
    out = torch.empty(rows, dtype=torch.int32, device=logits.device)
    fn = _function("sampling", "omnia_sample",
                   [c_void_p, c_longlong, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                    c_int, c_void_p, c_void_p, c_void_p, c_void_p])
    _check(fn(_ptr(logits), logits.stride(0), rows, vocab, _ptr(temperature), _ptr(top_k), _ptr(top_p), _ptr(min_p),
              _ptr(penalty), _ptr(history), 0 if history is None else history.shape[1], _ptr(seeds), _ptr(draws),
              _ptr(out), _stream()), "sample")
    return out


# ------------------------------------------------------------------------------------
# Residual streams, grouped norm and token shift (csrc/streams.cu)

MAX_STREAMS = 8


def embed_streams(ids: torch.Tensor, table: torch.Tensor, multiplier: float, streams: int) -> torch.Tensor:
    """x[t, s] = table[ids[t]] * multiplier for each of `streams` copies -> float32 [tokens, streams * hidden]."""
    tokens, (vocab, hidden) = ids.shape[0], table.shape
    x = torch.empty(tokens, streams * hidden, dtype=torch.float32, device=table.device)
    fn = _function("streams", "omnia_embed_streams",
                   [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_float, c_int, c_void_p, c_void_p])
    _check(fn(_ptr(ids), _ptr(table), _ptr(x), tokens, streams, hidden, vocab, multiplier, _code(table.dtype),
              _ptr(error_word(table.device)), _stream()), "embed_streams")
    return x


def streams_enter(xs: torch.Tensor, coef: torch.Tensor | None, streams: int, weight: torch.Tensor, eps: float,
                  groups: int, dtype: torch.dtype, step: StepContext | None = None, shift: torch.Tensor | None = None,
                  prev: torch.Tensor | None = None, last: torch.Tensor | None = None,
                  total: torch.Tensor | None = None) -> torch.Tensor:
    """h = norm(sum_s coef[s] xs[:, s]) with the RMS taken over `groups` equal runs of the width, then
    (with `shift`) h + (h_before - h) * shift, h_before being the token before's normed row: read from
    `prev` [slots, width] (by the step's state slots) for the first token of a request's portion. The
    last token of each portion leaves its normed row in `last` [requests, width] (float32), which
    `streams_leave` commits to `prev`. xs float32 [tokens, streams * width]; coef None means ones.
    `total` (float32 [tokens, width]), when given, receives the weighted sum of the streams itself."""
    tokens, width = xs.shape[0], xs.shape[1] // streams
    h = torch.empty(tokens, width, dtype=dtype, device=xs.device)
    fn = _function("streams", "omnia_streams_enter",
                   [c_void_p, c_void_p, c_int, c_int, c_void_p, c_float, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
                    c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_void_p])
    shifted = shift is not None
    _check(fn(_ptr(xs), _ptr(coef), streams, width, _ptr(weight), eps, groups, _ptr(shift),
              _ptr(prev) if shifted else None, _ptr(last) if shifted else None,
              _ptr(step.cu_seqlens) if shifted else None, _ptr(step.state_slots) if shifted else None,
              step.num_seqs if shifted else 0, _ptr(h), _ptr(total), tokens, _code(dtype), _stream()), "streams_enter")
    return h


def streams_leave(xs: torch.Tensor, branch: torch.Tensor, mix: torch.Tensor | None, out: torch.Tensor | None,
                  streams: int, step: StepContext | None = None, last: torch.Tensor | None = None,
                  prev: torch.Tensor | None = None, enter: tuple | None = None) -> torch.Tensor | None:
    """In place: xs[:, t] = sum_s mix[s, t] xs[:, s] + out[t] * branch for all t at once (`mix` None with
    one stream: xs += branch). With `last` and `prev`, every request's row of `last` is also copied
    into its state slot of `prev` (the token shift's commit). With `enter` = (coef, weight, eps,
    groups) the entry of the branch that follows (`streams_enter` without a shift) is done in the
    same kernel from the new streams, and its h is returned."""
    tokens, width = xs.shape[0], xs.shape[1] // streams
    commits = step.num_seqs if last is not None else 0
    h = torch.empty(tokens, width, dtype=branch.dtype, device=xs.device) if enter is not None else None
    coef, weight, eps, groups = enter if enter is not None else (None, None, 0.0, 1)
    fn = _function("streams", "omnia_streams_leave",
                   [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_int,
                    c_void_p, c_void_p, c_float, c_int, c_void_p, c_int, c_void_p])
    _check(fn(_ptr(xs), _ptr(branch), _ptr(mix), _ptr(out), streams, width, tokens, _ptr(last), _ptr(prev),
              _ptr(step.state_slots) if commits else None, commits, _ptr(coef), _ptr(weight), eps, groups, _ptr(h),
              _code(branch.dtype), _stream()), "streams_leave")
    return h


ACTIVATIONS = {"relu2": 0, "gelu_tanh": 1, "silu": 2}


def activation(z: torch.Tensor, kind: str) -> torch.Tensor:
    """relu(z)^2, the tanh form of GELU, or SiLU, element by element in float32."""
    act = torch.empty_like(z)
    fn = _function("elementwise", "omnia_activation", [c_void_p, c_void_p, c_longlong, c_int, c_int, c_void_p])
    _check(fn(_ptr(z), _ptr(act), z.numel(), ACTIVATIONS[kind], _code(z.dtype), _stream()), "activation")
    return act


def linear_act(a: torch.Tensor, weight: torch.Tensor, kind: str) -> torch.Tensor:
    """act(a @ weight^T): a few bfloat16 rows run on the weight-streaming kernel with the activation
    in its epilogue; otherwise the library's product and the activation kernel."""
    if _skinny(a, weight):
        out = torch.empty(a.shape[0], weight.shape[0], dtype=a.dtype, device=a.device)
        return _gemv_stream(a, weight, out, 0, 1.0, float(ACTIVATIONS[kind] + 1))
    return activation(_library_mm(a, weight), kind)


# ------------------------------------------------------------------------------------
# The gated delta rule and its short convolution (csrc/delta_rule.cu)

MAX_CONV_TAPS = 16


def short_conv(proj: torch.Tensor, col0: int, channels: int, taps: torch.Tensor, state: torch.Tensor,
               step: StepContext, unit_channels: int, unit_dim: int, unit_eps: float, scaled_channels: int,
               scale: float, a_rows: torch.Tensor | None = None, A_log: torch.Tensor | None = None,
               dt_bias: torch.Tensor | None = None, beta_col: int = 0, beta_heads: int = 0) -> torch.Tensor:
    """Everything of a recurrent mixer's token that needs no other token's result, one float32 row
    [y | decay | beta] a token (rows a multiple of 4 floats apart):
    y = silu(causal depth-wise convolution) of columns [col0, col0 + channels) of the projected rows,
    the inputs before a portion read from `state` [slots, taps - 1, channels]; the first
    `unit_channels` of y are made unit vectors in runs of `unit_dim`, the first `scaled_channels` of
    those also multiplied by `scale`; decay = exp(-exp(A_log[head]) softplus(a_rows + dt_bias)) per
    column of `a_rows` (heads x unit_dim); beta = sigmoid of the `beta_heads` columns of the projected
    rows from `beta_col`. The state is not moved on here (`delta_rule` does that)."""
    tokens = proj.shape[0]
    gates = a_rows.shape[1] if a_rows is not None else 0
    width = -(-(channels + gates + beta_heads) // 4) * 4
    y = torch.empty(tokens, width, dtype=torch.float32, device=proj.device)
    fn = _function("delta_rule", "omnia_short_conv",
                   [c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
                    c_float, c_int, c_float, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_int,
                    c_int, c_int, c_void_p], {"DELTA_DK": unit_dim})
    _check(fn(_ptr(proj), proj.shape[1], col0, channels, taps.shape[1], _ptr(taps), _ptr(state), _ptr(step.cu_seqlens),
              _ptr(step.state_slots), step.num_seqs, unit_channels, unit_dim, unit_eps, scaled_channels, scale,
              _ptr(a_rows), a_rows.stride(0) if a_rows is not None else 0, _ptr(A_log), _ptr(dt_bias), gates, beta_col,
              beta_heads, _ptr(y), width, tokens, _code(proj.dtype), _stream()), "short_conv")
    return y


def delta_parts(requests: int, heads: int, dv: int, sms: int, longest: int = 1 << 30) -> int:
    """Into how many runs of columns the recurrence kernel cuts a head's value channels: 1 (the block
    then also norms the head's output) when the step's (request, head) pairs give half the SMs a block
    each, or when no request brings more than 16 tokens (a decode step: measured at 8 requests of 8
    heads, 17 us whole against 37 us cut, which pays a second kernel and eight loads of q, k and the
    decays for one token); otherwise the fewest equal runs (of a multiple of 4 columns, at least 16)
    that give every SM about two blocks."""
    blocks = requests * heads
    if 2 * blocks >= sms or longest <= 16:
        return 1
    best = 1
    for parts in range(1, dv + 1):
        if dv % parts or (dv // parts) % 4 or dv // parts < 16:
            continue
        best = parts
        if blocks * parts >= 2 * sms:
            break
    return best


def delta_rule(conv: torch.Tensor, channels: int, groups: int, heads: int, dk: int, dv: int, proj: torch.Tensor,
               in_col: int, gate_rows: torch.Tensor, norm_weight: torch.Tensor, eps: float, S: torch.Tensor,
               conv_state: torch.Tensor, taps: int, step: StepContext, parts: int | None = None) -> torch.Tensor:
    """The gated delta rule with a decay per head and key channel over this step's tokens, request by
    request from the state in `S` [slots, heads, dk, dv] (float32, updated in place), followed by the
    RMS norm of each head's output, its weight and the sigmoid gate (`gate_rows` [tokens, heads * dv]
    logits). `conv` is `short_conv`'s output (q | k | v | decay | beta). Also moves `conv_state` on by
    this step's raw convolution inputs (columns from `in_col` of `proj`). -> [tokens, heads * dv]"""
    tokens = proj.shape[0]
    out = torch.empty(tokens, heads * dv, dtype=proj.dtype, device=proj.device)
    if parts is None:
        parts = delta_parts(step.num_seqs, heads, dv, sm_count(proj.device), step.max_q_len)
    raw = torch.empty(tokens, heads * dv, dtype=torch.float32, device=proj.device) if parts > 1 else None
    fn = _function("delta_rule", "omnia_delta_rule",
                   [c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_int, c_int, c_void_p, c_int,
                    c_void_p, c_float, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p,
                    c_int, c_void_p], {"DELTA_DK": dk})
    _check(fn(_ptr(conv), conv.shape[1], channels, groups, heads, dv, parts, _ptr(proj), proj.shape[1], in_col,
              _ptr(gate_rows), gate_rows.stride(0), _ptr(norm_weight), eps, _ptr(S), _ptr(conv_state), taps,
              _ptr(step.cu_seqlens), _ptr(step.state_slots), step.num_seqs, tokens, _ptr(out), _ptr(raw),
              _code(proj.dtype), _stream()), "delta_rule")
    return out


# ------------------------------------------------------------------------------------
# Linear attention with a constant decay per head (csrc/lightning.cu)


def lightning_parts(requests: int, heads: int, dv: int, sms: int) -> int:
    """Into how many runs of columns the recurrence kernel cuts a head's value channels: at least as
    many as bring a run down to 96 columns (four threads a column then fit a block; 192 and 384 where
    dv divides no better), and beyond that the fewest equal runs (of at least 8 columns) that give
    three quarters of the SMs a block when (request, head) pairs alone do not: every block stages its
    head's q and k for itself, so twice the blocks for the last quarter of the SMs is twice that work."""
    divisors = [parts for parts in range(1, dv + 1) if dv % parts == 0]
    least = next((parts for limit in (96, 192, 384) for parts in divisors if 8 <= dv // parts <= limit or
                  (dv // parts <= limit and parts == 1)), None)
    if least is None:
        least = next(parts for parts in divisors if dv // parts <= 96)
    blocks = requests * heads
    enough = sms - sms // 4
    best = least
    if blocks < enough:
        for parts in divisors:
            if parts < least or dv // parts < 8:
                continue
            best = parts
            if blocks * parts >= enough:
                break
    return best


def lightning_attention(proj: torch.Tensor, q_col: int, k_col: int, v_col: int, gate_col: int, heads: int, dk: int,
                        dv: int, decay: torch.Tensor, norm_weight: torch.Tensor, eps: float, S: torch.Tensor,
                        step: StepContext, parts: int | None = None) -> torch.Tensor:
    """Linear attention over this step's tokens, request by request from the state in `S`
    [slots, heads, dk, dv] (float32, updated in place): q, k, v = silu of the projected rows' columns
    from q_col, k_col (heads * dk each) and v_col (heads * dv); per head S <- decay_h S + k v^T,
    o = S^T q; then one RMS norm over a token's heads side by side (weight [heads * dv], `eps`) and the
    gate sigmoid(columns from gate_col). -> [tokens, heads * dv]"""
    tokens, stride = proj.shape
    width = heads * dv
    if parts is None:
        parts = lightning_parts(step.num_seqs, heads, dv, sm_count(proj.device))
    o_raw = torch.empty(tokens, width, dtype=torch.float32, device=proj.device)
    out = torch.empty(tokens, width, dtype=proj.dtype, device=proj.device)
    fn = _function("lightning", "omnia_lightning_recurrence",
                   [c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
                    c_int, c_void_p, c_int, c_void_p], {"LIGHTNING_DK": dk})
    _check(fn(_ptr(proj), stride, q_col, k_col, v_col, heads, dv, parts, _ptr(decay), _ptr(S), _ptr(step.cu_seqlens),
              _ptr(step.state_slots), step.num_seqs, _ptr(o_raw), _code(proj.dtype), _stream()), "lightning_recurrence")
    fn = _function("lightning", "omnia_lightning_out",
                   [c_void_p, c_void_p, c_int, c_void_p, c_float, c_int, c_int, c_void_p, c_int, c_void_p],
                   {"LIGHTNING_DK": dk})
    gate = proj.data_ptr() + gate_col * proj.element_size()
    _check(fn(_ptr(o_raw), gate, stride, _ptr(norm_weight), eps, width, tokens, _ptr(out), _code(proj.dtype), _stream()),
           "lightning_out")
    return out


def scaled_sum(a: torch.Tensor, sa: float, b: torch.Tensor, sb: float) -> torch.Tensor:
    """sa * a + sb * b, element by element, the sum in float32 and rounded once."""
    if a.shape != b.shape or a.dtype != b.dtype:
        raise KernelError("scaled_sum takes two tensors of one shape and type")
    out = torch.empty_like(a)
    fn = _function("elementwise", "omnia_scaled_sum",
                   [c_void_p, c_float, c_void_p, c_float, c_void_p, c_longlong, c_int, c_void_p])
    _check(fn(_ptr(a), sa, _ptr(b), sb, _ptr(out), a.numel(), _code(a.dtype), _stream()), "scaled_sum")
    return out


# ------------------------------------------------------------------------------------
# Linear attention with a decay per head or per key channel (csrc/state_recurrence.cu)


def state_columns(requests: int, heads: int, dk: int, dv: int, sms: int) -> int:
    """How many of a head's value columns a block of the recurrence kernel takes: at most 96 and no
    more than the key width leaves room for (a column needs enough threads that each holds at most 32
    rows of the state); a divisor of dv where it has one in reach, in fours where dv comes in fours; and
    halved, down to 8, while (request, head, run of columns) triples leave a quarter of the SMs idle: a
    prompt's tokens are walked one after another, so a lone prompt wants many narrow blocks."""
    threads = 1
    while -(-dk // threads) > 32:
        threads *= 2
    most = min(96, 448 // threads, dv)
    cols = next((c for c in range(most, most // 2, -1) if dv % c == 0 and (dv % 4 or c % 4 == 0)), most)
    if dv % 4 == 0:
        cols = max(4, cols // 4 * 4)
    while cols >= 16 and requests * heads * -(-dv // cols) < sms - sms // 4:
        cols = -(-cols // 2)
        if dv % 4 == 0:
            cols = -(-cols // 4) * 4
    return cols


def state_attention(proj: torch.Tensor, q_col: int, k_col: int, v_col: int, gate_col: int, heads: int, dk: int, dv: int,
                    S: torch.Tensor, step: StepContext, eps: float, decay: torch.Tensor | None = None,
                    decay_logits: torch.Tensor | None = None, decay_bias: torch.Tensor | None = None, tau: float = 1.0,
                    inv_freq: torch.Tensor | None = None, q_scale: float = 1.0, k_scale: float = 1.0,
                    norm_weight: torch.Tensor | None = None, gate: str = "silu",
                    cols: int | None = None, team: int = 0) -> torch.Tensor:
    """Linear attention over this step's tokens, request by request from the state in `S`
    [slots, heads, dk, dv] (float32, updated in place): per head S <- diag(a) S + k v^T, o = S^T q.
    q, k (heads * dk each) and v (heads * dv) are columns of the projected rows `proj`; q and k are
    turned over the first 2 * len(inv_freq) dims of every head in half-split pairs (float32 angles from
    the step's positions) and then multiplied by q_scale and k_scale, all in float32, and enter the
    recurrence unrounded. The decay is `decay` (float32 [heads], a constant a head) or, with
    `decay_logits` (float32 [tokens, heads * dk]), a = sigmoid(logits + decay_bias)^(1 / tau) per token
    and key channel. Every head's o is divided by its own root mean square (`eps` inside the root), multiplied
    by `norm_weight` ([dv], shared by the heads; None: no weight) and by silu or sigmoid (`gate`) of the
    columns from gate_col. `cols`: value columns a block takes; `team`: threads a column (0: the kernel's
    choice). -> [tokens, heads * dv]"""
    tokens, stride = proj.shape
    if (decay is None) == (decay_logits is None):
        raise KernelError("state_attention takes either a decay per head or decay logits per token")
    if gate not in ("silu", "sigmoid"):
        raise KernelError(f"state_attention gates by silu or sigmoid, not {gate!r}")
    channel = decay_logits is not None
    if channel and decay_logits.dtype != torch.float32:
        decay_logits = decay_logits.float()
    defines = {"STATE_DK": dk}
    width = heads * dv
    rot = 0 if inv_freq is None else 2 * inv_freq.shape[0]
    if step.decode_only and cols is None and 4 * (3 * dk + max(1024 // dv, 1) * dv) <= 40 * 1024:
        # Single tokens: the input step, the recurrence and the heads' norm and gate in one kernel.
        out = torch.empty(tokens, width, dtype=proj.dtype, device=proj.device)
        fn = _function("state_recurrence", "omnia_state_step",
                       [c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_int, c_void_p, c_float,
                        c_float, c_void_p, c_int, c_void_p, c_float, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p,
                        c_float, c_int, c_void_p, c_int, c_void_p], defines)
        _check(fn(_ptr(proj), stride, q_col, k_col, v_col, gate_col, heads, dv, _ptr(inv_freq), rot, _ptr(step.positions),
                  q_scale, k_scale, _ptr(decay_logits), decay_logits.stride(0) if channel else 0, _ptr(decay_bias), 1.0 / tau,
                  _ptr(decay), _ptr(S), _ptr(step.cu_seqlens), _ptr(step.state_slots), step.num_seqs, _ptr(norm_weight), eps,
                  int(gate == "silu"), _ptr(out), _code(proj.dtype), _stream()), "state_step")
        return out
    if cols is None:
        cols = state_columns(step.num_seqs, heads, dk, dv, sm_count(proj.device))
    row_floats = 2 * (-(-heads * dk // 4) * 4) + -(-width // 4) * 4 + (-(-heads * dk // 4) * 4 if channel else 0)
    rows = torch.empty(tokens, row_floats, dtype=torch.float32, device=proj.device)
    fn = _function("state_recurrence", "omnia_state_inputs",
                   [c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_int, c_void_p, c_float, c_float,
                    c_void_p, c_int, c_void_p, c_float, c_void_p, c_int, c_int, c_void_p], defines)
    _check(fn(_ptr(proj), stride, q_col, k_col, v_col, heads, dv, _ptr(inv_freq), rot, _ptr(step.positions), q_scale,
              k_scale, _ptr(decay_logits), decay_logits.stride(0) if channel else 0, _ptr(decay_bias), 1.0 / tau, _ptr(rows),
              tokens, _code(proj.dtype), _stream()), "state_inputs")
    o_raw = torch.empty(tokens, width, dtype=torch.float32, device=proj.device)
    fn = _function("state_recurrence", "omnia_state_recurrence",
                   [c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p,
                    c_int, c_void_p], defines)
    _check(fn(_ptr(rows), heads, dv, cols, int(channel), _ptr(decay), _ptr(S), _ptr(step.cu_seqlens),
              _ptr(step.state_slots), step.num_seqs, _ptr(o_raw), team, _stream()), "state_recurrence")
    out = torch.empty(tokens, width, dtype=proj.dtype, device=proj.device)
    fn = _function("state_recurrence", "omnia_state_heads_out",
                   [c_void_p, c_void_p, c_int, c_void_p, c_float, c_int, c_int, c_int, c_int, c_void_p, c_int, c_void_p],
                   defines)
    _check(fn(_ptr(o_raw), proj.data_ptr() + gate_col * proj.element_size(), stride, _ptr(norm_weight), eps, heads, dv,
              tokens, int(gate == "silu"), _ptr(out), _code(proj.dtype), _stream()), "state_heads_out")
    return out


# ------------------------------------------------------------------------------------
# A real-gated linear recurrence over channels behind a short convolution (csrc/rglru.cu)

RGLRU_MAX_TAPS = 16
RGLRU_SCAN_WARPS = 16


def gated_channel_recurrence(proj: torch.Tensor, x_col: int, y_col: int, x_bias: torch.Tensor | None,
                             y_bias: torch.Tensor | None, taps: torch.Tensor, conv_bias: torch.Tensor | None,
                             gates: torch.Tensor, r_bias: torch.Tensor, i_bias: torch.Tensor, lam: torch.Tensor,
                             c_decay: float, S: torch.Tensor, conv_state: torch.Tensor, step: StepContext,
                             warps: int | None = None) -> torch.Tensor:
    """The recurrence S_t = a_t S_(t-1) + sqrt(1 - a_t^2) i_t u_t over `channels` independent channels,
    request by request from `S` [slots, channels] (float32, updated in place), with
    u = a causal convolution (`taps` [channels, K], the last column the current token's; `conv_bias`) of
    x = proj[:, x_col:] + x_bias continued from `conv_state` [slots, K - 1, channels] (the request's last
    inputs, moved on); r, i = sigmoid of block-diagonal maps of u (`gates` float32 [blocks, width,
    2 * width]: r's columns, then i's; a batched vendor product in true float32) plus `r_bias`, `i_bias`;
    a = exp(-c_decay * r * softplus(lam)). Everything from x on is float32.
    -> S_t * gelu_tanh(proj[:, y_col:] + y_bias) as [tokens, channels] in proj's type."""
    tokens, stride = proj.shape
    C, K = taps.shape
    blocks, bw = gates.shape[0], gates.shape[1]
    if blocks * bw != C or gates.shape[2] != 2 * bw or not 1 <= K <= RGLRU_MAX_TAPS:
        raise KernelError(f"a recurrence over {C} channels in {blocks} blocks of {bw}, {K} taps")
    device, code = proj.device, _code(proj.dtype)
    if step.decode_only and 5 * bw * 4 <= 40 * 1024:
        # Single tokens: the convolution, the gates' maps and the recurrence in one kernel.
        out = torch.empty(tokens, C, dtype=proj.dtype, device=device)
        fn = _function("rglru", "omnia_rglru_step",
                       [c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                        c_void_p, c_float, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int,
                        c_void_p])
        _check(fn(_ptr(proj), stride, x_col, y_col, _ptr(x_bias), _ptr(y_bias), _ptr(taps), _ptr(conv_bias), _ptr(gates),
                  _ptr(r_bias), _ptr(i_bias), _ptr(lam), c_decay, C, bw, K, _ptr(S), _ptr(conv_state), _ptr(step.cu_seqlens),
                  _ptr(step.state_slots), step.num_seqs, _ptr(out), code, _stream()), "rglru_step")
        return out
    u = torch.empty(tokens, C, dtype=torch.float32, device=device)
    fn = _function("rglru", "omnia_rglru_conv",
                   [c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_int,
                    c_void_p, c_int, c_int, c_void_p])
    _check(fn(_ptr(proj), stride, x_col, _ptr(x_bias), _ptr(taps), _ptr(conv_bias), C, K, _ptr(conv_state),
              _ptr(step.cu_seqlens), _ptr(step.state_slots), step.num_seqs, _ptr(u), tokens, code, _stream()), "rglru_conv")
    z = batched_mm(u.view(tokens, blocks, bw).transpose(0, 1), gates)  # [blocks, tokens, 2 bw]
    a, b, y = (torch.empty(tokens, C, dtype=torch.float32, device=device) for _ in range(3))
    fn = _function("rglru", "omnia_rglru_gates",
                   [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_float, c_void_p, c_int, c_int, c_void_p, c_int, c_int,
                    c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p])
    _check(fn(_ptr(u), _ptr(z), _ptr(r_bias), _ptr(i_bias), _ptr(lam), c_decay, _ptr(proj), stride, y_col, _ptr(y_bias), C,
              bw, tokens, _ptr(a), _ptr(b), _ptr(y), code, _stream()), "rglru_gates")
    if warps is None:
        warps = max(1, min(RGLRU_SCAN_WARPS, step.max_q_len // 32))
    out = torch.empty(tokens, C, dtype=proj.dtype, device=device)
    fn = _function("rglru", "omnia_rglru_scan",
                   [c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p,
                    c_void_p, c_void_p, c_int, c_int, c_void_p, c_int, c_void_p])
    _check(fn(_ptr(a), _ptr(b), _ptr(y), C, K, _ptr(S), _ptr(conv_state), _ptr(proj), stride, x_col, _ptr(x_bias),
              _ptr(step.cu_seqlens), _ptr(step.state_slots), step.num_seqs, warps, _ptr(out), code, _stream()), "rglru_scan")
    return out


# ------------------------------------------------------------------------------------
# Attention over a latent cache (csrc/attention_latent.cu)

LATENT_MAX_RANK = 512


def latent_prepare(proj: torch.Tensor, q_col: int, heads: int, q_dim: int, down_col: int, rank: int, rot: int,
                   weight: torch.Tensor, eps: float, inv_freq: torch.Tensor, positions: torch.Tensor,
                   kv: KVView) -> None:
    """Per projected row: the RMS-normed latent (columns [down_col, down_col + rank)) and the rotated
    shared key part (the `rot` columns after it) go to the row's cache slot; the last `rot` dims of
    each of the `heads` query heads (each `q_dim` wide, from `q_col`) are rotated in place. The rotation
    pairs dims (2i, 2i + 1) over the first 2 * len(inv_freq) of the `rot`."""
    store = kv.writes
    fn = _function("attention_latent", "omnia_latent_prepare",
                   [c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_float, c_void_p, c_int,
                    c_void_p, c_void_p, c_void_p, c_longlong, c_int, c_int, c_void_p, c_void_p])
    _check(fn(_ptr(proj), proj.shape[1], q_col, heads, q_dim, down_col, rank, rot, _ptr(weight), eps, _ptr(inv_freq),
              2 * inv_freq.shape[0], _ptr(positions), _ptr(kv.slot_mapping) if store else None, _ptr(kv.pages),
              kv.pages.shape[0] * kv.page_size, proj.shape[0], _code(proj.dtype), _ptr(error_word(proj.device)),
              _stream()), "latent_prepare")


def latent_tc_supported(q_lat: torch.Tensor, q_rot: torch.Tensor, out: torch.Tensor, scale: float) -> bool:
    """The tensor-core kernel takes bfloat16, a latent that is a multiple of 64 wide, a row (latent
    and rotated part) that is a multiple of 32, a positive scale, and operands whose rows start on
    16 bytes."""
    rank, rot = q_lat.shape[2], q_rot.shape[2]
    return (q_lat.dtype == torch.bfloat16 and rank % 64 == 0 and (rank + rot) % 32 == 0 and scale > 0
            and all(t.stride(0) % 8 == 0 and t.stride(1) % 8 == 0 and t.data_ptr() % 16 == 0
                    for t in (q_lat, q_rot, out)))


def latent_split_plan(q_lens, heads: int, longest: int, rows_per_block: int, sms: int) -> tuple[int, int]:
    """(splits, keys per split) of the tensor-core latent attention kernel: one split while the step's
    row blocks fill the GPU; otherwise the keys are cut (in multiples of 32, at least 128 a split) so
    that about two blocks run on every SM."""
    blocks = sum(-(-q * heads // rows_per_block) for q in q_lens)
    if blocks >= sms or longest <= 128:
        return 1, 0
    splits = min(-(-2 * sms // blocks), -(-longest // 128), 256)
    chunk = -(-(-(-longest // splits)) // 32) * 32
    return -(-longest // chunk), chunk


def latent_attention(q_lat: torch.Tensor, q_rot: torch.Tensor, kv: KVView, step: StepContext, scale: float,
                     sink: torch.Tensor | None, gate: torch.Tensor | None, out: torch.Tensor,
                     tensor_cores: bool | None = None) -> torch.Tensor:
    """Causal attention of every head over the cache's latent rows (see csrc/attention_latent.cu).
    q_lat [heads, tokens, rank], q_rot [tokens, heads, rot] and out [heads, tokens, rank] may be
    strided views (last dim contiguous); gate [tokens, >= heads] holds one logit per head in its
    first columns; sink float32 [heads]. bfloat16 of supported widths runs on the tensor-core kernel
    (csrc/attention_latent_tc.cu; `tensor_cores` False keeps it off), everything else, the 32-bit
    path among it, on the generic one."""
    heads, tokens, rank = q_lat.shape
    rot = q_rot.shape[2]
    if q_lat.stride(2) != 1 or q_rot.stride(2) != 1 or out.stride(2) != 1 or (gate is not None and gate.stride(1) != 1):
        raise KernelError("latent_attention wants the last dim of its operands contiguous")
    if tensor_cores is not False and latent_tc_supported(q_lat, q_rot, out, scale):
        most_rows = step.max_q_len * heads
        groups = 4 if most_rows > 32 else 2 if most_rows > 16 else 1
        defines = {"LATENT_RANK": rank, "LATENT_ROT": rot, "LATENT_ROW_GROUPS": groups}
        # The bound on a request's length that is fixed for a captured step: its block table's width.
        longest = kv.block_table.shape[1] * kv.page_size
        splits, chunk = latent_split_plan(step.q_lens, heads, longest, 16 * groups, sm_count(q_lat.device))
        part_o = part_ml = None
        if splits > 1:
            part_o, part_ml = _step_buffers(step, q_lat.device, {
                "latent_part_o": (tokens * heads * splits * rank, torch.float32, False),
                "latent_part_ml": (tokens * heads * splits * 2, torch.float32, False)})
        fn = _function("attention_latent_tc", "omnia_latent_attention_tc",
                       [c_void_p, c_longlong, c_longlong, c_void_p, c_longlong, c_longlong, c_void_p, c_void_p, c_void_p,
                        c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_longlong, c_longlong, c_void_p, c_void_p,
                        c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_void_p,
                        c_void_p], defines)
        _check(fn(_ptr(q_lat), q_lat.stride(0), q_lat.stride(1), _ptr(q_rot), q_rot.stride(1), q_rot.stride(0),
                  _ptr(kv.pages), _ptr(kv.block_table), _ptr(step.cu_seqlens), _ptr(step.seq_lens), _ptr(sink),
                  _ptr(gate), gate.stride(0) if gate is not None else 0, _ptr(out), out.stride(0), out.stride(1),
                  _ptr(part_o), _ptr(part_ml), tokens, step.num_seqs, step.max_q_len, kv.block_table.shape[1],
                  kv.pages.shape[0], heads, kv.page_size, kv.window or 0, splits, chunk, scale,
                  _ptr(error_word(q_lat.device)), _stream()), "latent_attention_tc")
        return out
    if rank > LATENT_MAX_RANK:
        raise KernelError(f"latent_attention takes a latent of at most {LATENT_MAX_RANK}, got {rank}")
    fn = _function("attention_latent", "omnia_latent_attention",
                   [c_void_p, c_longlong, c_longlong, c_void_p, c_longlong, c_longlong, c_void_p, c_void_p, c_void_p,
                    c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_longlong, c_longlong, c_int, c_int, c_int, c_int,
                    c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_void_p, c_void_p])
    _check(fn(_ptr(q_lat), q_lat.stride(0), q_lat.stride(1), _ptr(q_rot), q_rot.stride(1), q_rot.stride(0),
              _ptr(kv.pages), _ptr(kv.block_table), _ptr(step.cu_seqlens), _ptr(step.positions), _ptr(sink),
              _ptr(gate), gate.stride(0) if gate is not None else 0, _ptr(out), out.stride(0), out.stride(1), tokens,
              step.num_seqs, kv.block_table.shape[1], kv.pages.shape[0], heads, rank, rot, kv.page_size,
              kv.window or 0, scale, _code(q_lat.dtype), _ptr(error_word(q_lat.device)), _stream()),
           "latent_attention")
    return out


def batched_mm(a: torch.Tensor, b: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    """a [batch, rows, k] times b [batch, k, n] -> [batch, rows, n]: the vendor library's strided
    batched product (float32 accumulation; true float32 on the 32-bit path)."""
    if a.dtype == torch.float32 and (torch.backends.cuda.matmul.allow_tf32
                                      or torch.get_float32_matmul_precision() != "highest"):
        raise KernelError("the 32-bit path needs true float32 matrix products; TF32 is switched on")
    return torch.bmm(a, b) if out is None else torch.bmm(a, b, out=out)


# ------------------------------------------------------------------------------------
# Routed experts (csrc/moe.cu)


def moe_route(h: torch.Tensor, router: torch.Tensor, correction: torch.Tensor | None, experts: int, top: int,
              counts: torch.Tensor, scoring: str = "softmax") -> tuple[torch.Tensor, torch.Tensor]:
    """Per row of `h`: float32 logits against `router` (float32 [outputs, hidden]), softmax over all
    outputs (or, with `scoring` "sigmoid", every output's own sigmoid), the `top` largest of score +
    correction; -> (choice int32 [rows, top], weight float32
    [rows, top]: the chosen outputs' scores, not renormalised). Outputs at or beyond `experts` are identity experts; the
    others are counted into `counts` (int32 [experts], zero before the call)."""
    rows, hidden = h.shape
    choice = torch.empty(rows, top, dtype=torch.int32, device=h.device)
    weight = torch.empty(rows, top, dtype=torch.float32, device=h.device)
    if scoring not in ("softmax", "sigmoid"):
        raise KernelError(f"router scores are a softmax or sigmoids, not {scoring!r}")
    fn = _function("moe", "omnia_moe_route",
                   [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p,
                    c_int, c_void_p])
    _check(fn(_ptr(h), _ptr(router), _ptr(correction), rows, router.shape[0], experts, hidden, top,
              int(scoring == "sigmoid"), _ptr(choice), _ptr(weight), _ptr(counts), _code(h.dtype), _stream()), "moe_route")
    return choice, weight


def moe_route_table(token_ids: torch.Tensor, table: torch.Tensor, experts: int,
                    counts: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """Routing by a table instead of a router: row `token_ids[t]` of `table` (int32 [vocab, top]) names
    token t's experts, each with the weight 1 / top; -> (choice int32 [rows, top], weight float32
    [rows, top]), the choices counted into `counts` (int32 [experts], zero before the call)."""
    rows, (vocab, top) = token_ids.shape[0], table.shape
    choice = torch.empty(rows, top, dtype=torch.int32, device=table.device)
    weight = torch.empty(rows, top, dtype=torch.float32, device=table.device)
    fn = _function("moe", "omnia_moe_route_table",
                   [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p])
    _check(fn(_ptr(token_ids), _ptr(table), rows, vocab, experts, top, _ptr(choice), _ptr(weight), _ptr(counts),
              _ptr(error_word(table.device)), _stream()), "moe_route_table")
    return choice, weight


MOE_TILE_ROWS = 64
"""Rows of a tile of the grouped products of csrc/moe.cu (the tcgen05 kernel's grouped form takes 128)."""

MOE_TCGEN05_PAIRS = 1024
"""From this many (row, choice) pairs on, and at least 64 of them an expert on average, the bfloat16
grouped products run on the tcgen05 kernel (tiles of 128 rows of one expert each; fewer rows an expert
would leave most of every tile empty); below, on the mma.sync kernel with tiles of 64 rows."""


def moe_experts(h: torch.Tensor, router: torch.Tensor | None, correction: torch.Tensor | None, gate_up: torch.Tensor,
                down: torch.Tensor, top: int, step: StepContext | None = None,
                tensor_cores: bool | None = None, tcgen05: bool | None = None,
                table: torch.Tensor | None = None, token_ids: torch.Tensor | None = None,
                alpha: float = 1.0, limit: float = 0.0, scoring: str = "softmax", weigh: str = "output",
                extra: torch.Tensor | None = None) -> torch.Tensor:
    """A routed mixture of gated feed-forward experts over the rows of `h` [rows, hidden]:
    y = sum over a row's `top` choices of score * expert(h), expert e being
    down[e] (silu(gate_e h) * (up_e h)) with gate_up [experts, 2 inner, hidden] (gate rows, then up
    rows) and down [experts, hidden, inner]; router outputs beyond the experts with tensors are
    identity experts (their output is h). Nothing is asked of the host: rows are sorted by expert on
    the device, and the grouped products walk a tile list made there. bfloat16 runs on the tensor
    cores: the tcgen05 kernel's grouped form for many rows (`tcgen05` names the choice), mma.sync for
    few (`tensor_cores` False keeps both off); float32 on the ordinary cores.

    With `table` (int32 [vocab, top]) and the rows' `token_ids` there is no router: a token's experts are
    its id's row of the table, each weighing 1 / top. `limit` > 0 makes every expert the clamped unit
    g = min(gate h, limit), u = clamp(up h, -limit, limit), down(g sigmoid(alpha g) (u + 1)).
    `scoring`: the router's scores are a "softmax" over all outputs or every output's own "sigmoid".
    `weigh` "input": y = sum of expert(score * h) instead: a choice's score multiplies what its expert
    is given (the product in float32, rounded once), and the experts' outputs are added as they are.
    `extra` [rows, hidden]: added to y in the same pass (an expert that every row uses)."""
    if weigh not in ("output", "input"):
        raise KernelError(f"a choice's weight goes on its expert's output or input, not {weigh!r}")
    rows, hidden = h.shape
    experts, inner = gate_up.shape[0], gate_up.shape[1] // 2
    pairs = rows * top
    device = h.device
    if step is None:
        step = _NoStep()
    if tensor_cores is None:
        tensor_cores = h.dtype == torch.bfloat16 and hidden % 8 == 0 and inner % 8 == 0
    if tcgen05 is None:
        tcgen05 = tensor_cores and pairs >= MOE_TCGEN05_PAIRS and pairs >= 64 * experts
    tile_rows = 128 if tcgen05 else MOE_TILE_ROWS
    max_tiles = min(pairs, -(-pairs // tile_rows) + experts)
    counts, cursors = _step_buffers(step, device, {"moe_counts": (experts, torch.int32, True),
                                                   "moe_cursors": (experts, torch.int32, True)})
    if table is not None:
        choice, weight = moe_route_table(token_ids[:rows], table, experts, counts)
    else:
        choice, weight = moe_route(h, router, correction, experts, top, counts, scoring)
    ints = torch.empty(2 * pairs + experts + 1 + 3 * max_tiles + 1, dtype=torch.int32, device=device)
    place, source = ints[:pairs], ints[pairs: 2 * pairs]
    offsets = ints[2 * pairs: 2 * pairs + experts + 1]
    tiles = ints[2 * pairs + experts + 1: 2 * pairs + experts + 1 + 3 * max_tiles]
    tile_count = ints[-1:]
    fn = _function("moe", "omnia_moe_plan",
                   [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
                    c_int, c_int, c_void_p])
    _check(fn(_ptr(choice), _ptr(counts), _ptr(cursors), _ptr(offsets), _ptr(tiles), _ptr(tile_count), _ptr(place),
              _ptr(source), rows, top, experts, max_tiles, tile_rows, _stream()), "moe_plan")
    act = torch.empty(pairs, inner, dtype=h.dtype, device=device)
    out = torch.empty(pairs, hidden, dtype=h.dtype, device=device)
    sorted_rows = None
    if weigh == "input":
        # The weighted rows in sorted order; rows past the last sorted one (identity choices) stay unread.
        sorted_rows = torch.empty(pairs, hidden, dtype=h.dtype, device=device)
        fn = _function("moe", "omnia_moe_weighted_rows",
                       [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p])
        _check(fn(_ptr(h), _ptr(place), _ptr(weight), _ptr(sorted_rows), pairs, hidden, top, _code(h.dtype), _stream()),
               "moe_weighted_rows")
    if tcgen05:
        if sorted_rows is None:
            sorted_rows = torch.empty(pairs, hidden, dtype=h.dtype, device=device)
            fn = _function("moe", "omnia_moe_gather", [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p])
            _check(fn(_ptr(h), _ptr(source), _ptr(offsets[experts:]), _ptr(sorted_rows), pairs, hidden, _code(h.dtype),
                      _stream()), "moe_gather")
        grouped = _function("gemm_tcgen05", "omnia_gemm_tcgen05_grouped",
                            [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_int,
                             c_float, c_float, c_void_p, c_void_p])
        err = _ptr(error_word(device))
        _check(grouped(_ptr(sorted_rows), _ptr(gate_up), _ptr(act), pairs, 2 * inner, hidden, experts, 1, _ptr(tiles),
                       _ptr(tile_count), max_tiles, alpha, limit, err, _stream()), "gemm_tcgen05_grouped")
        _check(grouped(_ptr(act), _ptr(down), _ptr(out), pairs, hidden, inner, experts, 0, _ptr(tiles),
                       _ptr(tile_count), max_tiles, 1.0, 0.0, err, _stream()), "gemm_tcgen05_grouped")
    else:
        product = _function("moe", "omnia_moe_product",
                            [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                             c_float, c_float, c_int, c_int, c_void_p])
        _check(product(_ptr(h if sorted_rows is None else sorted_rows), _ptr(source) if sorted_rows is None else None,
                       _ptr(gate_up), _ptr(act), _ptr(tiles), _ptr(tile_count), max_tiles, inner,
                       hidden, 1, alpha, limit, _code(h.dtype), int(tensor_cores), _stream()), "moe_product")
        _check(product(_ptr(act), None, _ptr(down), _ptr(out), _ptr(tiles), _ptr(tile_count), max_tiles, hidden, inner, 0,
                       1.0, 0.0, _code(h.dtype), int(tensor_cores), _stream()), "moe_product")
    y = torch.empty_like(h)
    fn = _function("moe", "omnia_moe_combine",
                   [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p])
    _check(fn(_ptr(out), _ptr(h), _ptr(place), _ptr(weight) if weigh == "output" else None, _ptr(extra), _ptr(y), rows,
              hidden, top, _code(h.dtype), _stream()), "moe_combine")
    return y


class _NoStep:
    """Stands in for a step where an op is called on its own (tests of single kernels)."""
    workspace = None
