"""Python bindings of the CUDA kernels: argument checks, then a ctypes call on
the current stream.  Every function works on CUDA tensors only and raises if
the kernels' library is missing or the GPU is absent: there is no CPU path.
"""
import ctypes

import torch

from . import build

F32, BF16 = 0, 1
ACT = {None: 0, "none": 0, "gelu_tanh": 1, "gelu_erf": 2, "xielu": 3, "relu2": 4}
ACT_SLOTS = 256              # parameter slots per kernel library (common.cuh: SGLC_ACT_SLOTS)
_act_slots = []              # slot -> (a, b), as registered
_act_synced = {}             # library name -> slots already written into it


def _act(act):
    """The integer a launcher takes: the kind, and for ("xielu", slot) the slot in the next byte."""
    if isinstance(act, tuple):
        return ACT[act[0]] | (int(act[1]) << 8)
    if act == "xielu":
        raise KernelError("xielu needs its parameters: pass (\"xielu\", slot) from register_act_params()")
    return ACT[act]


def register_act_params(a, b, libraries):
    """Give the two numbers of an activation a slot in the parameter tables of the named kernel
    libraries (equal numbers share a slot) and return it, or None when the tables are full (the
    caller then applies the activation with a kernel of its own).  Done when a model is loaded,
    never inside a step: the copy into a library's table synchronises."""
    pair = (float(a), float(b))
    if pair in _act_slots:
        slot = _act_slots.index(pair)
    elif len(_act_slots) < ACT_SLOTS:
        _act_slots.append(pair)
        slot = len(_act_slots) - 1
    else:
        return None
    for name in libraries:
        lib = build.load(name)
        done = _act_synced.get((name, id(lib)), 0)
        for i in range(done, len(_act_slots)):
            code = lib.sglc_set_act_params(i, ctypes.c_float(_act_slots[i][0]), ctypes.c_float(_act_slots[i][1]))
            if code != 0:
                raise KernelError(f"{name}: setting activation parameters failed (code {code})")
        _act_synced[(name, id(lib))] = len(_act_slots)
    return slot
_DT = {torch.float32: F32, torch.bfloat16: BF16}


# how many kernels of this package were launched (bench and tests read it)
LAUNCHES = 0


class KernelError(RuntimeError):
    pass


def _ptr(t):
    return ctypes.c_void_p(t.data_ptr() if t is not None else 0)


_PINNED_STREAM = None


# Set by profile_begin(): a list of (label, start event, end event), one per launch.  Every
# binding below evaluates _stream() just before its launch and _check() just after, so the two
# bracket the kernel.
_PROFILE = None
_PROFILE_START = None


def _stream():
    global _PROFILE_START
    if _PROFILE is not None:
        _PROFILE_START = torch.cuda.Event(enable_timing=True)
        _PROFILE_START.record()
    if _PINNED_STREAM is not None:
        return _PINNED_STREAM
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def profile_begin():
    """From here on every kernel launch of this package is bracketed by a pair of CUDA events
    (which also keeps a kernel from starting under the one ahead: the times are the kernels'
    own, not their share of an overlapped step).  Queue the work behind something long, so that
    the host's launch cost does not show between the events."""
    global _PROFILE
    _PROFILE = []


def profile_end():
    """{kernel label: (launches, microseconds)} since profile_begin(); synchronises."""
    global _PROFILE
    rows, _PROFILE = _PROFILE, None
    torch.cuda.synchronize()
    out = {}
    for label, e0, e1 in rows or []:
        n, us = out.get(label, (0, 0.0))
        out[label] = (n + 1, us + e0.elapsed_time(e1) * 1e3)
    return out


class pinned_stream:
    """Within the block every kernel goes to the stream that is current at entry, looked up
    once (the lookup costs as much as a launch; a forward pass makes a hundred)."""

    def __enter__(self):
        global _PINNED_STREAM
        self.before = _PINNED_STREAM
        _PINNED_STREAM = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)

    def __exit__(self, *exc):
        global _PINNED_STREAM
        _PINNED_STREAM = self.before


def _dt(t, what):
    try:
        return _DT[t.dtype]
    except KeyError:
        raise KernelError(f"{what}: dtype {t.dtype} is not handled (float32 or bfloat16)") from None


UNSUPPORTED = -2      # a launcher's "size not supported by this kernel"


def _need_cuda(*tensors):
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise KernelError("kernels run on CUDA tensors only; got a CPU tensor "
                              "(this engine has no CPU path)")


def _check(lib, code, what, n_kernels=1):
    global LAUNCHES
    LAUNCHES += n_kernels
    if _PROFILE is not None and _PROFILE_START is not None:
        end = torch.cuda.Event(enable_timing=True)
        end.record()
        _PROFILE.append((what.split(" ")[0], _PROFILE_START, end))
    if code != 0:
        msg = lib.sglc_error_string(code).decode()
        raise KernelError(f"{what}: {msg} (code {code})")


def _i32(t, what):
    if t.dtype != torch.int32 or not t.is_contiguous():
        raise KernelError(f"{what} must be a contiguous int32 tensor")


# ---------------------------------------------------------------------------
def embed(tokens, table, out, positions=None, pos_table=None, err_flag=None, inv_freq=None):
    """out[t,:] = table[tokens[t],:] (+ pos_table[positions[t],:]); out is float32 [T,E].
    With inv_freq (float64 [ceil(E/2)]) instead of a position table, the sinusoidal vector
    sin/cos(positions[t] * inv_freq[i]) at entries 2i / 2i+1 is added."""
    _need_cuda(tokens, table, out, positions, pos_table, inv_freq)
    _i32(tokens, "tokens")
    T, E = out.shape
    if out.dtype != torch.float32 or not out.is_contiguous():
        raise KernelError("embed: out must be contiguous float32")
    if table.shape[1] != E or not table.is_contiguous():
        raise KernelError(f"embed: table {tuple(table.shape)} does not match width {E}")
    if inv_freq is not None:
        _i32(positions, "positions")
        if pos_table is not None or inv_freq.dtype != torch.float64 or inv_freq.numel() != (E + 1) // 2 \
                or not inv_freq.is_contiguous():
            raise KernelError("embed: inverse wavelengths must be float64, one per pair of columns, and come "
                              "without a position table")
        lib = build.load("embed")
        code = lib.sglc_embed_sinusoid(_ptr(tokens), _ptr(positions), _ptr(table), _ptr(inv_freq), _ptr(out),
                                       T, E, table.shape[0], _dt(table, "embed table"), _ptr(err_flag), _stream())
        _check(lib, code, "embed_sinusoid")
        return
    P = 0
    if pos_table is not None:
        _i32(positions, "positions")
        if pos_table.dtype != table.dtype or pos_table.shape[1] != E or not pos_table.is_contiguous():
            raise KernelError("embed: position table must have the token table's dtype and width")
        P = pos_table.shape[0]
    lib = build.load("embed")
    code = lib.sglc_embed(_ptr(tokens), _ptr(positions), _ptr(table), _ptr(pos_table), _ptr(out),
                          T, E, table.shape[0], P, _dt(table, "embed table"), _ptr(err_flag), _stream())
    _check(lib, code, "embed")


def add_rows(x, idx, table):
    """x[t,:] += table[idx[t],:] (x float32)."""
    _need_cuda(x, idx, table)
    _i32(idx, "idx")
    T, E = x.shape
    if x.dtype != torch.float32 or not x.is_contiguous() or table.shape[1] != E:
        raise KernelError("add_rows: x must be contiguous float32 of the table's width")
    lib = build.load("embed")
    code = lib.sglc_add_rows(_ptr(x), _ptr(idx), _ptr(table), T, E, table.shape[0],
                             _dt(table, "table"), _stream())
    _check(lib, code, "add_rows")


def layernorm(x, gamma, beta, eps, out, rows=None):
    """out[r,:] = LayerNorm(x[rows[r] or r,:]); x float32 [*,E]; out float32 or bfloat16."""
    _need_cuda(x, gamma, beta, out, rows)
    E = x.shape[-1]
    n = out.shape[0]
    if x.dtype != torch.float32 or not x.is_contiguous() or not out.is_contiguous():
        raise KernelError("layernorm: x must be contiguous float32 and out contiguous")
    if gamma.dtype != torch.float32 or beta.dtype != torch.float32 or gamma.numel() != E or beta.numel() != E:
        raise KernelError("layernorm: gain and bias must be float32 vectors of the row width")
    if rows is not None:
        _i32(rows, "rows")
        if rows.numel() < n:
            raise KernelError("layernorm: fewer row indices than output rows")
    elif x.shape[0] < n:
        raise KernelError("layernorm: fewer input rows than output rows")
    lib = build.load("layernorm")
    code = lib.sglc_layernorm(_ptr(x), _ptr(rows), _ptr(gamma), _ptr(beta), _ptr(out), n, E,
                              ctypes.c_float(eps), _dt(out, "layernorm out"), _stream())
    _check(lib, code, f"layernorm (width {E})")


def gemm_simt(a, w, bias, out=None, residual=None, act=None):
    """out = act(a·wᵀ + bias), or residual += a·wᵀ + bias.  a [M,K] (row stride free),
    w [N,K] contiguous; plain FFMA with 32-bit accumulation."""
    _need_cuda(a, w, bias, out, residual)
    M, K = a.shape
    N = w.shape[0]
    if w.shape[1] != K or not w.is_contiguous() or a.stride(1) != 1 or a.dtype != w.dtype:
        raise KernelError(f"gemm: a {tuple(a.shape)}/{a.dtype} and w {tuple(w.shape)}/{w.dtype} do not match")
    if bias is not None and (bias.dtype != torch.float32 or bias.numel() != N):
        raise KernelError("gemm: bias must be a float32 vector of N")
    dst = residual if residual is not None else out
    if dst is None or dst.shape[0] < M or dst.shape[1] != N or dst.stride(1) != 1:
        raise KernelError("gemm: output does not match [M,N]")
    if residual is not None and residual.dtype != torch.float32:
        raise KernelError("gemm: the residual stream is float32")
    lib = build.load("gemm_simt")
    code = lib.sglc_gemm_simt(_ptr(a), _ptr(w), _ptr(bias), _ptr(out), _ptr(residual), M, N, K,
                              a.stride(0), dst.stride(0), _dt(a, "gemm input"),
                              _dt(dst, "gemm output"), _act(act), _stream())
    _check(lib, code, f"gemm_simt M={M} N={N} K={K}")


def kv_write(k_src, v_src, cache, slots, n_kv_heads, head_dim):
    """Scatter keys and values of T tokens into one layer's pages.
    k_src, v_src: [T, n_kv_heads*head_dim] views (row stride free); cache:
    [n_pages, 2, n_kv_heads, page_size, head_dim]; slots int32 [T]."""
    _need_cuda(k_src, v_src, cache, slots)
    _i32(slots, "slots")
    T = k_src.shape[0]
    n_pages, two, H, page_size, D = cache.shape
    if two != 2 or H != n_kv_heads or D != head_dim or not cache.is_contiguous():
        raise KernelError(f"kv_write: cache {tuple(cache.shape)} does not match heads {n_kv_heads} x {head_dim}")
    if k_src.shape[1] != H * D or k_src.stride(1) != 1 or v_src.stride(1) != 1 \
            or k_src.stride(0) != v_src.stride(0) or k_src.dtype != cache.dtype:
        raise KernelError("kv_write: key/value rows do not match the cache")
    lib = build.load("kv_cache")
    code = lib.sglc_kv_write(_ptr(k_src), _ptr(v_src), k_src.stride(0), _ptr(cache), _ptr(slots), T,
                             H, D, page_size, n_pages, _dt(k_src, "kv source"), _dt(cache, "cache"),
                             _stream())
    _check(lib, code, "kv_write")


def attention_simt(q, cache, block_table, token_req, positions, out, n_heads, scale, window,
                   max_keys, max_q_len=None, kv_shared=False):
    """Causal attention of T tokens over the paged cache, 32-bit arithmetic.
    q: [T, n_heads*head_dim] view; out likewise; block_table int32 [R, max_blocks].
    max_q_len: the longest portion among the tokens (1 when every request brings one token;
    unknown: None); it only decides how many tokens share a block.
    kv_shared: cache is [n_pages, 1, n_kv_heads, page_size, head_dim], rows that are keys and
    values at once."""
    _need_cuda(q, cache, block_table, token_req, positions, out)
    for t, nm in ((block_table, "block_table"), (token_req, "token_req"), (positions, "positions")):
        _i32(t, nm)
    T = q.shape[0]
    n_pages, two, Hkv, page_size, D = cache.shape
    if q.shape[1] != n_heads * D or q.stride(1) != 1 or out.stride(1) != 1 or q.dtype != out.dtype:
        raise KernelError("attention: query/output rows do not match heads x head_dim")
    if q.dtype != cache.dtype:
        raise KernelError("attention: queries and cache must have one dtype")
    if two != (1 if kv_shared else 2):
        raise KernelError(f"attention: cache {tuple(cache.shape)} does not fit kv_shared={kv_shared}")
    lib = build.load("attention_simt")
    fn = lib.sglc_attention_simt_shared if kv_shared else lib.sglc_attention_simt
    code = fn(_ptr(q), q.stride(0), _ptr(cache), _ptr(block_table),
              block_table.stride(0), _ptr(token_req), _ptr(positions), _ptr(out),
              out.stride(0), T, n_heads, Hkv, D, page_size, ctypes.c_float(scale),
              int(window or 0), int(max_keys), _dt(q, "attention q"),
              _dt(cache, "cache"), n_pages, _ptr(tc_error_flag(q.device)),
              int(max_q_len) if max_q_len else 2, _stream())
    _check(lib, code, f"attention_simt (head_dim {D}, up to {max_keys} keys)")


# ---------------------------------------------------------------------------
# tensor-core GEMM (bfloat16, tcgen05 + TMA)
_tc_scratch = {}
TC_WS_FLOATS = 8 << 20          # 32 MB of split-K partial sums
TC_COUNTERS = 8192


def _tc_buffers(device):
    """Split-K workspace, tile counters (zero between launches) and the error word of the
    tensor-core kernels, one set per device, allocated at first use."""
    b = _tc_scratch.get(device)
    if b is None:
        b = (torch.empty(TC_WS_FLOATS, dtype=torch.float32, device=device),
             torch.zeros(TC_COUNTERS, dtype=torch.int32, device=device),
             torch.zeros(1, dtype=torch.int32, device=device))
        _tc_scratch[device] = b
    return b


def tc_error_flag(device):
    return _tc_buffers(device)[2]


def wait_probe(device, polls=300, peer_cycles=200000):
    """Makes a bounded wait run out, on purpose and harmlessly: two tiny kernels (csrc/wait_probe.cu)
    wait, with a limit of `polls`, on barriers that nobody arrives on, give up, tear down as the
    tensor-core kernels do and set the error word those kernels share.  Returns the kernels' trace
    [waiter, its block's other warps, cluster waiter, peer left, waiter left] (2 = ran out,
    1 = happened); the error word is left set for the caller to find."""
    lib = build.load("wait_probe")
    err = _tc_buffers(torch.device(device))[2]
    trace = torch.zeros(5, dtype=torch.int32, device=device)
    code = lib.sglc_wait_probe(_ptr(err), _ptr(trace), ctypes.c_uint(int(polls)), int(peer_cycles), _stream())
    _check(lib, code, "wait_probe", n_kernels=2)
    return trace.tolist()


def gemm_tc_supported(a, w):
    """TMA needs 16-byte aligned rows: K and the row stride multiples of 8 elements."""
    return (a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and a.dim() == 2
            and a.shape[1] % 8 == 0 and a.stride(1) == 1 and a.stride(0) % 8 == 0
            and a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0 and w.is_contiguous())


def gemm_tc(a, w, bias, out=None, residual=None, act=None, supported=False):
    """out = act(a·wᵀ + bias) (bfloat16 or float32), or residual += a·wᵀ + bias, on the
    tensor cores.  a [M,K] bfloat16 (row stride free), w [N,K] bfloat16 contiguous.
    supported=True: the caller has just asked gemm_tc_supported(a, w)."""
    _need_cuda(a, w, bias, out, residual)
    if not supported and not gemm_tc_supported(a, w):
        raise KernelError(f"gemm_tc: operands a {tuple(a.shape)} stride {a.stride()} / w {tuple(w.shape)} "
                          "do not meet the 16-byte row rule of TMA (K and row stride multiples of 8)")
    M, K = a.shape
    N = w.shape[0]
    if w.shape[1] != K:
        raise KernelError(f"gemm_tc: a {tuple(a.shape)} and w {tuple(w.shape)} do not match")
    if bias is not None and (bias.dtype != torch.float32 or bias.numel() != N):
        raise KernelError("gemm_tc: bias must be a float32 vector of N")
    dst = residual if residual is not None else out
    if dst is None or dst.shape[0] < M or dst.shape[1] != N or dst.stride(1) != 1:
        raise KernelError("gemm_tc: output does not match [M,N]")
    if residual is not None:
        if residual.dtype != torch.float32:
            raise KernelError("gemm_tc: the residual stream is float32")
        if act not in (None, "none"):
            raise KernelError("gemm_tc: no activation when adding into the residual stream")
    elif dst.dtype not in (torch.float32, torch.bfloat16):
        raise KernelError("gemm_tc: output must be float32 or bfloat16")
    lib = build.load("gemm_tc")
    err = _tc_buffers(a.device)[2]
    code = lib.sglc_gemm_tc(_ptr(a), _ptr(w), _ptr(bias), _ptr(out), _ptr(residual), M, N, K,
                            a.stride(0), dst.stride(0), 1 if dst.dtype == torch.float32 else 0,
                            _act(act), _ptr(err), _stream())
    _check(lib, code, f"gemm_tc M={M} N={N} K={K}")


def gemm_tc_kv(a, w, bias, out, cache, slots, n_heads, n_kv_heads, head_dim):
    """The query/key/value projection of a step with prompt portions, with the cache write in its
    epilogue: out[:, :n_heads*head_dim] takes the queries; keys and values go straight into the
    paged cache [n_pages, 2, n_kv_heads, page_size, head_dim] at slots[token].  Returns False,
    having launched nothing, when the product would not take the many-token kernel or the sizes
    do not fall on its tiles (the caller then projects and writes the cache separately)."""
    _need_cuda(a, w, bias, out, cache, slots)
    M, K = a.shape
    N = w.shape[0]
    if not gemm_tc_supported(a, w) or w.shape[1] != K or out.dtype != torch.bfloat16 or cache.dtype != torch.bfloat16 \
            or out.shape[1] != N or out.stride(1) != 1 or not cache.is_contiguous() \
            or N != (n_heads + 2 * n_kv_heads) * head_dim:
        return False
    _i32(slots, "slots")
    n_pages, two, Hkv, page_size, D = cache.shape
    if two != 2 or Hkv != n_kv_heads or D != head_dim or slots.numel() < M:
        raise KernelError("gemm_tc_kv: the cache or the slots do not match the projection")
    lib = build.load("gemm_tc")
    err = _tc_buffers(a.device)[2]
    code = lib.sglc_gemm_tc_kv(_ptr(a), _ptr(w), _ptr(bias), _ptr(out), M, N, K, a.stride(0), out.stride(0), ACT[None],
                               _ptr(cache), _ptr(slots), n_heads * head_dim, n_kv_heads, head_dim, page_size, n_pages,
                               _ptr(err), _stream())
    if code == UNSUPPORTED:
        return False
    _check(lib, code, f"gemm_tc_kv M={M} N={N} K={K}")
    return True


def gemm_tc_form(M, N, K, act=None):
    """Which of gemm_tc's kernels a product of these sizes takes: "few" (up to 128 tokens: weights on
    the MMA's 128-row side, split-K over a cluster), "stream" (many tokens, one block a tile) or "pair"
    (many tokens on pairs of SMs)."""
    return ("few", "stream", "pair")[build.load("gemm_tc").sglc_gemm_tc_form(int(M), int(N), int(K), _act(act))]


FEW_MAX_TOKENS = 2           # products of so few tokens go to gemm_few ...
FEW_MAX_WEIGHT = 3 << 20     # ... if the weight matrix has no more elements than this


def gemm_few(a, w, bias, out=None, residual=None, act=None):
    """The same product as gemm_tc for up to 8 tokens: 8 output features a block over the whole
    of K, operands from global memory straight into the registers of the warp-level
    tensor-core instruction, no block waiting for another."""
    _need_cuda(a, w, bias, out, residual)
    M, K = a.shape
    N = w.shape[0]
    lib = build.load("gemm_few")
    if w.shape[1] != K or not gemm_tc_supported(a, w) or not lib.sglc_gemm_few_supports(M, N, K, a.stride(0)):
        raise KernelError(f"gemm_few: a {tuple(a.shape)} stride {a.stride()} / w {tuple(w.shape)}: up to 8 "
                          "tokens, K and the row stride multiples of 8, 16-byte aligned operands")
    if bias is not None and (bias.dtype != torch.float32 or bias.numel() != N):
        raise KernelError("gemm_few: bias must be a float32 vector of N")
    dst = residual if residual is not None else out
    if dst is None or dst.shape[0] < M or dst.shape[1] != N or dst.stride(1) != 1:
        raise KernelError("gemm_few: output does not match [M,N]")
    if residual is not None:
        if residual.dtype != torch.float32:
            raise KernelError("gemm_few: the residual stream is float32")
        if act not in (None, "none"):
            raise KernelError("gemm_few: no activation when adding into the residual stream")
    elif dst.dtype not in (torch.float32, torch.bfloat16):
        raise KernelError("gemm_few: output must be float32 or bfloat16")
    code = lib.sglc_gemm_few(_ptr(a), _ptr(w), _ptr(bias), _ptr(out), _ptr(residual), M, N, K,
                             a.stride(0), dst.stride(0), 1 if dst.dtype == torch.float32 else 0,
                             _act(act), _stream())
    _check(lib, code, f"gemm_few M={M} N={N} K={K}")


# ---------------------------------------------------------------------------
STREAM_MIN_ITEMS = 160     # (token, head) items from which the streaming decode kernel is used
USE_TMA_DECODE = True      # tests switch it off to reach the register-staged kernel at head size 64/128


def attention_decode(q, cache, block_table, token_req, positions, out, n_heads, scale, window,
                     max_keys, k_new=None, v_new=None, slots=None, token_list=None, n_tokens=None,
                     n_splits=None, variant=None):
    """Attention of single decoded tokens over the paged bfloat16 cache, keys split across
    blocks and merged in a fixed order.  With k_new/v_new/slots (the step's own keys and
    values, [T, n_kv_heads*head_dim] views, and their cache slots) the same launch also writes
    them into the cache; this is valid only when every request brings exactly one token.
    `token_list` (int32, its first `n_tokens` entries) names the tokens to serve; a list of all
    tokens is an order in which the streaming kernel takes them (long contexts first balance
    its blocks).
    Three kernels serve it, chosen by the size of the launch (or named by `variant`, for tests
    and tuning: "stream", "tma", "register")."""
    _need_cuda(q, cache, block_table, token_req, positions, out, k_new, v_new, slots, token_list)
    for t, nm in ((block_table, "block_table"), (positions, "positions")):
        _i32(t, nm)
    if token_req is not None:           # None: token t belongs to the step's t-th request
        _i32(token_req, "token_req")
    T = q.shape[0]
    order_only = False
    if token_list is not None:          # serve only the listed tokens (the first n_tokens entries)
        _i32(token_list, "token_list")
        if token_req is None or k_new is not None:
            # without a token -> request table, or with the cache write, the list can only be an
            # order of all tokens (long ones first); the streaming kernel alone makes use of it
            if int(n_tokens) != T:
                raise KernelError("attention_decode: a list of some tokens needs token_req and no fused cache write")
            order_only = True
        T = int(n_tokens)
    n_pages, two, Hkv, page_size, D = cache.shape
    if q.dtype != torch.bfloat16 or cache.dtype != torch.bfloat16 or out.dtype != torch.bfloat16:
        raise KernelError("attention_decode: bfloat16 queries, cache and output only")
    if q.shape[1] != n_heads * D or q.stride(1) != 1 or out.stride(1) != 1:
        raise KernelError("attention_decode: query/output rows do not match heads x head_dim")
    lib = build.load("attention_decode")
    ws, counters, err = _tc_buffers(q.device)
    splits = int(n_splits) if n_splits else lib.sglc_attention_decode_splits(T, n_heads, int(max_keys))
    need_ws, need_c = ctypes.c_longlong(0), ctypes.c_int(0)
    lib.sglc_attention_decode_scratch(T, n_heads, D, splits, ctypes.byref(need_ws), ctypes.byref(need_c))
    if need_ws.value > ws.numel() or need_c.value > counters.numel():
        splits = 1
    new_stride = 0
    if k_new is not None:
        _i32(slots, "slots")
        if v_new is None or k_new.dtype != torch.bfloat16 or tuple(k_new.shape) != (T, Hkv * D) \
                or k_new.stride(1) != 1 or v_new.stride(1) != 1 or k_new.stride(0) != v_new.stride(0):
            raise KernelError("attention_decode: new keys/values do not match the cache")
        new_stride = k_new.stride(0)
    if variant not in (None, "stream", "tma", "register"):
        raise KernelError(f"attention_decode: unknown variant {variant!r}")
    if variant == "stream" or (variant is None and USE_TMA_DECODE and T * n_heads >= STREAM_MIN_ITEMS):
        # many (token, head) items: resident blocks stream them through a ring of TMA stages
        tlib = build.load("attention_decode_tma")
        if tlib.sglc_attention_decode_stream_supports(D, page_size, int(max_keys), int(window or 0)) \
                and (page_size * D * 2) % 128 == 0:
            code = tlib.sglc_attention_decode_stream(_ptr(q), q.stride(0), _ptr(cache), _ptr(block_table),
                                                     block_table.stride(0), _ptr(token_req), _ptr(positions),
                                                     _ptr(out), out.stride(0), T, n_heads, Hkv, D, page_size,
                                                     ctypes.c_float(scale), int(window or 0), int(max_keys),
                                                     _ptr(k_new), _ptr(v_new), new_stride, _ptr(slots),
                                                     _ptr(err), _ptr(token_list), n_pages, _stream())
            _check(tlib, code, f"attention_decode_stream (head_dim {D}, up to {max_keys} keys)")
            return
        if variant == "stream":
            raise KernelError(f"attention_decode_stream does not take head_dim {D}, page size {page_size}, "
                              f"{max_keys} keys")
    if order_only:
        token_list = None
    if D in (64, 128) and splits <= 8 and (page_size * D * 2) % 128 == 0 and page_size <= 256 \
            and ((variant is None and USE_TMA_DECODE and T * n_heads * splits <= 1536) or variant == "tma"):
        # keys and values staged through shared memory by TMA (measured faster up to about a
        # thousand blocks; beyond, the register-staged kernel is a few percent ahead)
        tlib = build.load("attention_decode_tma")
        code = tlib.sglc_attention_decode_tma(_ptr(q), q.stride(0), _ptr(cache), _ptr(block_table),
                                              block_table.stride(0), _ptr(token_req), _ptr(positions),
                                              _ptr(out), out.stride(0), T, n_heads, Hkv, D, page_size,
                                              ctypes.c_float(scale), int(window or 0), int(max_keys), splits,
                                              _ptr(k_new), _ptr(v_new), new_stride, _ptr(slots), _ptr(err),
                                              _ptr(token_list), n_pages, _stream())
        if code != -2 or variant == "tma":  # -2: the range does not fit its shared memory; use the other kernel
            _check(tlib, code, f"attention_decode_tma (head_dim {D}, up to {max_keys} keys)")
            return
    code = lib.sglc_attention_decode(_ptr(q), q.stride(0), _ptr(cache), _ptr(block_table),
                                     block_table.stride(0), _ptr(token_req), _ptr(positions), _ptr(out),
                                     out.stride(0), T, n_heads, Hkv, D, page_size, ctypes.c_float(scale),
                                     int(window or 0), int(max_keys), splits, _ptr(ws), _ptr(counters),
                                     _ptr(k_new), _ptr(v_new), new_stride, _ptr(slots), _ptr(err),
                                     _ptr(token_list), n_pages, _stream())
    _check(lib, code, f"attention_decode (head_dim {D}, up to {max_keys} keys)")


def attention_decode_shared(q, cache, block_table, token_req, positions, out, n_heads, scale, window, max_keys,
                            token_list=None, n_tokens=None):
    """Attention of single decoded tokens over a bfloat16 cache [n_pages, 1, n_kv_heads, page_size,
    head_dim] whose rows are keys and values at once (a latent), keys split across blocks and
    merged in a fixed order; the rows of the step's own tokens are in the cache already.
    token_req None: token t belongs to the step's t-th request.  token_list (int32, its first
    n_tokens entries; needs token_req): the tokens to serve."""
    _need_cuda(q, cache, block_table, token_req, positions, out, token_list)
    for t, nm in ((block_table, "block_table"), (positions, "positions")):
        _i32(t, nm)
    T = q.shape[0]
    if token_req is not None:
        _i32(token_req, "token_req")
    if token_list is not None:
        _i32(token_list, "token_list")
        if token_req is None:
            raise KernelError("attention_decode_shared: a list of some tokens needs token_req")
        T = int(n_tokens)
    n_pages, one, Hkv, page_size, D = cache.shape
    if one != 1 or q.dtype != torch.bfloat16 or cache.dtype != torch.bfloat16 or out.dtype != torch.bfloat16:
        raise KernelError("attention_decode_shared: bfloat16 queries, output and cache [n_pages,1,heads,page,dim]")
    if q.shape[1] != n_heads * D or q.stride(1) != 1 or out.stride(1) != 1:
        raise KernelError("attention_decode_shared: query/output rows do not match heads x head_dim")
    lib = build.load("attention_decode")
    ws, counters, err = _tc_buffers(q.device)
    splits = lib.sglc_attention_decode_splits(T, n_heads, int(max_keys))
    need_ws, need_c = ctypes.c_longlong(0), ctypes.c_int(0)
    lib.sglc_attention_decode_scratch(T, n_heads, D, splits, ctypes.byref(need_ws), ctypes.byref(need_c))
    if need_ws.value > ws.numel() or need_c.value > counters.numel():
        splits = 1
    code = lib.sglc_attention_decode_shared(_ptr(q), q.stride(0), _ptr(cache), _ptr(block_table),
                                            block_table.stride(0), _ptr(token_req), _ptr(positions), _ptr(out),
                                            out.stride(0), T, n_heads, Hkv, D, page_size, ctypes.c_float(scale),
                                            int(window or 0), int(max_keys), splits, _ptr(ws), _ptr(counters),
                                            _ptr(err), _ptr(token_list), n_pages, _stream())
    _check(lib, code, f"attention_decode_shared (head_dim {D}, up to {max_keys} keys)")


def attention_latent_decode_supported(q, cache, n_heads):
    """Whether the all-heads-a-block kernel takes this cache and these queries."""
    n_pages, one, Hkv, page_size, D = cache.shape
    return (one == 1 and Hkv == 1 and q.dtype == torch.bfloat16 and cache.dtype == torch.bfloat16
            and bool(build.load("attention_latent").sglc_attention_latent_decode_supports(int(n_heads), int(D))))


def attention_latent_decode(q, cache, block_table, token_req, positions, out, n_heads, scale, window, max_keys,
                            token_list=None, n_tokens=None, n_splits=None):
    """Attention of single decoded tokens over a cached latent [n_pages, 1, 1, page_size, D] (rows
    that are keys and values of every head): one block serves all heads of a token over a range
    of its keys, so a row comes from memory once.  token_req None: token t belongs to the step's
    t-th request.  token_list (int32, its first n_tokens entries): the tokens to serve."""
    _need_cuda(q, cache, block_table, token_req, positions, out, token_list)
    for t, nm in ((block_table, "block_table"), (positions, "positions")):
        _i32(t, nm)
    T = q.shape[0]
    if token_req is not None:
        _i32(token_req, "token_req")
    if token_list is not None:
        _i32(token_list, "token_list")
        T = int(n_tokens)
    n_pages, one, Hkv, page_size, D = cache.shape
    if one != 1 or Hkv != 1 or not cache.is_contiguous() or cache.dtype != torch.bfloat16 \
            or q.dtype != torch.bfloat16 or out.dtype != torch.bfloat16:
        raise KernelError("attention_latent_decode: bfloat16 queries and output, cache [n_pages,1,1,page,dim]")
    if q.shape[1] != n_heads * D or q.stride(1) != 1 or out.stride(1) != 1:
        raise KernelError("attention_latent_decode: query/output rows do not match heads x dim")
    lib = build.load("attention_latent")
    ws, _, err = _tc_buffers(q.device)
    splits = int(n_splits) if n_splits else lib.sglc_attention_latent_decode_splits(T, int(max_keys))
    if splits > 1 and T * splits * n_heads * (D + 2) > ws.numel():
        splits = 1
    code = lib.sglc_attention_latent_decode(_ptr(q), q.stride(0), _ptr(cache), _ptr(block_table),
                                            block_table.stride(0), _ptr(token_req), _ptr(positions), _ptr(token_list),
                                            _ptr(out), out.stride(0), T, n_heads, D, page_size, ctypes.c_float(scale),
                                            int(window or 0), splits, _ptr(ws), ctypes.c_longlong(ws.numel()), n_pages,
                                            _ptr(err), _stream())
    _check(lib, code, f"attention_latent_decode (dim {D}, up to {max_keys} keys)", n_kernels=2 if splits > 1 else 1)


# ---------------------------------------------------------------------------
def attention_prefill_tc_supported(q, cache, scale):
    D = cache.shape[-1]
    return (q.dtype == torch.bfloat16 and cache.dtype == torch.bfloat16 and D in (64, 128)
            and scale > 0 and q.stride(0) % 8 == 0 and q.data_ptr() % 16 == 0)


def attention_prefill_tc(q, cache, block_table, q_start, kv_len, out, n_heads, scale, window,
                         n_requests, max_q_len, skip_single=False, kv_shared=False, chunk=None, sinks=None):
    """Causal attention of prompt portions on the tensor cores (tcgen05), bfloat16, head
    sizes 64 and 128.  q_start int32 [R+1], kv_len int32 [R] (lengths after this step).
    kv_shared: cache is [n_pages, 1, n_kv_heads, page_size, head_dim], rows that are keys and
    values at once.  chunk: a query sees only the keys of its own chunk of so many positions;
    sinks: float32 [n_heads], a score per head that joins the softmax's denominator."""
    _need_cuda(q, cache, block_table, q_start, kv_len, out, sinks)
    for t, nm in ((block_table, "block_table"), (q_start, "q_start"), (kv_len, "kv_len")):
        _i32(t, nm)
    n_pages, two, Hkv, page_size, D = cache.shape
    if not attention_prefill_tc_supported(q, cache, scale):
        raise KernelError(f"attention_prefill_tc: head size {D} / dtype {q.dtype} / scale {scale} not "
                          "supported (bfloat16, head size 64 or 128, positive scale)")
    if q.shape[1] != n_heads * D or q.stride(1) != 1 or out.stride(1) != 1 or out.dtype != torch.bfloat16 \
            or out.stride(0) % 8 != 0 or out.data_ptr() % 16 != 0:
        raise KernelError("attention_prefill_tc: query/output rows do not match heads x head_dim")
    if two != (1 if kv_shared else 2):
        raise KernelError(f"attention_prefill_tc: cache {tuple(cache.shape)} does not fit kv_shared={kv_shared}")
    lib = build.load("attention_prefill_tc")
    err = _tc_buffers(q.device)[2]
    if chunk or sinks is not None:
        if kv_shared or (sinks is not None and (sinks.dtype != torch.float32 or sinks.numel() != n_heads)):
            raise KernelError("attention_prefill_tc: a chunk mask or sinks go with separate keys and values; "
                              "one float32 sink per head")
        code = lib.sglc_attention_prefill_tc_ext(
            _ptr(q), q.stride(0), _ptr(cache), _ptr(block_table), block_table.stride(0), _ptr(q_start), _ptr(kv_len),
            _ptr(out), out.stride(0), int(n_requests), int(max_q_len), n_heads, Hkv, D, page_size,
            ctypes.c_float(scale), int(window or 0), int(chunk or 0), _ptr(sinks), q.shape[0], n_pages,
            1 if skip_single else 0, _ptr(err), _stream())
        _check(lib, code, f"attention_prefill_tc (head_dim {D}, chunk {chunk})")
        return
    fn = lib.sglc_attention_prefill_tc_shared if kv_shared else lib.sglc_attention_prefill_tc
    code = fn(_ptr(q), q.stride(0), _ptr(cache), _ptr(block_table),
              block_table.stride(0), _ptr(q_start), _ptr(kv_len), _ptr(out),
              out.stride(0), int(n_requests), int(max_q_len), n_heads, Hkv, D,
              page_size, ctypes.c_float(scale), int(window or 0), q.shape[0],
              n_pages, 1 if skip_single else 0, _ptr(err), _stream())
    _check(lib, code, f"attention_prefill_tc (head_dim {D})")


# ---------------------------------------------------------------------------
def sample(logits, params, hist_tok, hist_cnt, out_tok, out_logprob=None):
    """One token per row of `logits` ([n, V] float32, row stride free; penalties
    change the rows in place).  `params`: int32 tensor [n, 10] holding the packed
    per-row records (see sampling.cu); hist_tok/hist_cnt: int32 (token, count)
    pairs of the rows' histories."""
    _need_cuda(logits, params, hist_tok, hist_cnt, out_tok, out_logprob)
    n, V = logits.shape
    if logits.dtype != torch.float32 or logits.stride(1) != 1:
        raise KernelError("sample: logits must be float32 rows")
    if params.dtype != torch.int32 or params.shape != (n, 10) or not params.is_contiguous():
        raise KernelError("sample: params must be a contiguous int32 [n,10] tensor")
    _i32(out_tok, "out_tok")
    lib = build.load("sampling")
    code = lib.sglc_sample(_ptr(logits), logits.stride(0), V, n, _ptr(params), _ptr(hist_tok),
                           _ptr(hist_cnt), _ptr(out_tok), _ptr(out_logprob), _stream())
    _check(lib, code, "sample")


# ---------------------------------------------------------------------------
NORM_FORMS = {"layer": 0, "rms": 1, "copy": 2}      # "copy": norm_add_tail's `then` stage only


def norm_rows(src, gain, bias, eps, dst, form="layer", add=False, dst_rows=None, src_rows=None, groups=1):
    """dst[r,:] = norm(src[r,:]) * gain + bias (gain, bias: float32 vectors or None), `form`
    "layer" (mean removed) or "rms"; src float32 or bfloat16 [n,E] with a free row stride.
    groups > 1: a row is `groups` equal consecutive parts, each normalised by its own statistics
    (gain and bias still span the row).
    add=True: dst (float32) += the normalised rows.  dst_rows (int32 [n]): row r goes to
    dst[dst_rows[r], :] (dst [rows, E]: the rows of a paged cache seen flat).  src_rows (int32):
    output row r is made from src[src_rows[r], :]; as many rows as dst has (or dst_rows names)."""
    _need_cuda(src, gain, bias, dst, dst_rows, src_rows)
    n, E = src.shape
    if src_rows is not None:
        _i32(src_rows, "src_rows")
        n = dst.shape[0] if dst_rows is None else dst_rows.numel()
        if src_rows.numel() < n:
            raise KernelError("norm_rows: fewer source row indices than output rows")
    if src.stride(1) != 1 or dst.stride(-1) != 1 or dst.shape[-1] != E or dst.dim() != 2:
        raise KernelError("norm_rows: rows must be contiguous and of one width")
    for v, nm in ((gain, "gain"), (bias, "bias")):
        if v is not None and (v.dtype != torch.float32 or v.numel() != E or not v.is_contiguous()):
            raise KernelError(f"norm_rows: {nm} must be a float32 vector of the row width")
    if dst_rows is not None:
        _i32(dst_rows, "dst_rows")
        if dst_rows.numel() < n:
            raise KernelError("norm_rows: fewer destination rows than source rows")
    elif dst.shape[0] < n:
        raise KernelError("norm_rows: fewer destination rows than source rows")
    if add and dst.dtype != torch.float32:
        raise KernelError("norm_rows: the sum goes into a float32 destination")
    if groups < 1 or E % groups:
        raise KernelError(f"norm_rows: a row of {E} does not split into {groups} equal parts")
    lib = build.load("norm_rows")
    code = lib.sglc_norm_rows_grouped(_ptr(src), ctypes.c_longlong(src.stride(0)), _dt(src, "norm source"),
                                      _ptr(src_rows), _ptr(gain),
                                      _ptr(bias), _ptr(dst), ctypes.c_longlong(dst.stride(0)),
                                      _dt(dst, "norm destination"), _ptr(dst_rows), ctypes.c_longlong(dst.shape[0]), n,
                                      E, ctypes.c_float(eps), NORM_FORMS[form], 1 if add else 0, int(groups),
                                      _ptr(tc_error_flag(src.device)), _stream())
    _check(lib, code, f"norm_rows (width {E})")


def norm_add_tail(y, gain, eps, x, form="layer", mix=None, then=None):
    """x += norm(y) * gain (x: float32 [T,E], the residual stream; y float32 [T,E]); then, in the same
    launch, mix = (hist, n_terms, weights): hist[n_terms-1] = x, x = sum_j weights[j] * hist[j]
    (as depth_mix), and then = (gain, eps, form, out): out = norm(x) * gain (the norm ahead of the
    next sublayer; form "copy" with gain None: out = x in out's precision, for a sublayer that reads
    the stream itself).  The bits are those of the separate kernels."""
    hist, n_terms, weights = mix if mix is not None else (None, 0, None)
    g2, eps2, form2, out = then if then is not None else (None, 0.0, "layer", None)
    _need_cuda(y, gain, x, hist, weights, g2, out)
    n, E = y.shape
    if y.dtype != torch.float32 or x.dtype != torch.float32 or y.stride(1) != 1 or not x.is_contiguous() \
            or x.shape[1] != E or x.shape[0] < n:
        raise KernelError("norm_add_tail: y and x are float32 [T,E], x contiguous")
    if hist is not None and (hist.dtype != torch.float32 or not hist.is_contiguous() or hist.shape[0] < n_terms
                             or tuple(hist.shape[1:]) != (n, E)):
        raise KernelError("norm_add_tail: hist is float32 [>= n_terms, T, E] for this step's T")
    if out is not None and (tuple(out.shape) != (n, E) or out.stride(1) != 1):
        raise KernelError("norm_add_tail: the next norm's output is [T,E]")
    if form == "copy" or (form2 == "copy") != (then is not None and g2 is None):
        raise KernelError("norm_add_tail: \"copy\" is the second stage's form, and goes without a gain")
    lib = build.load("norm_rows")
    code = lib.sglc_norm_add_tail(_ptr(y), ctypes.c_longlong(y.stride(0)), _ptr(gain), ctypes.c_float(eps),
                                  NORM_FORMS[form], _ptr(x), _ptr(hist),
                                  ctypes.c_longlong(n * E), int(n_terms), _ptr(weights), _ptr(g2),
                                  ctypes.c_float(eps2), NORM_FORMS[form2], _ptr(out),
                                  ctypes.c_longlong(out.stride(0) if out is not None else 0),
                                  _dt(out, "norm output") if out is not None else F32, n, E, _stream())
    _check(lib, code, f"norm_add_tail (width {E})")


GATED_SCAN_CHUNK = 128      # a step whose longest portion exceeds this goes the gated scans' chunked way ...
GATED_SCAN_PIECE = 32       # ... in pieces of so many tokens a block (gated_scan.cu: SCAN_CHUNK, SCAN_PIECE)


def mingru_scan_workspace(n_requests, width, n_tokens, max_q_len):
    """Floats of workspace mingru_scan needs for such a step: none while the longest portion fits
    one chunk, else two per channel and piece row plus one per channel and request."""
    if max_q_len <= GATED_SCAN_CHUNK:
        return 0
    return int(width) * (2 * (int(n_tokens) // GATED_SCAN_PIECE + int(n_requests)) + int(n_requests))


def mingru_scan(gate, cand, out_gate, y, state, q_start, state_slots, n_requests, max_q_len, workspace=None):
    """The minGRU recurrence over the step's tokens (see gated_scan.cu).  gate, cand, out_gate:
    float32 [T,W] column ranges of one buffer; y: [T,W] float32 or bfloat16; state: float32
    [n_slots, W], read and written in place for the requests' slots."""
    _need_cuda(gate, cand, out_gate, y, state, q_start, state_slots, workspace)
    T, W = gate.shape
    for t in (gate, cand, out_gate):
        if t.dtype != torch.float32 or tuple(t.shape) != (T, W) or t.stride(1) != 1 or t.stride(0) != gate.stride(0):
            raise KernelError("mingru_scan: gate, candidate and output gate must be float32 [T,W] of one row stride")
    if tuple(y.shape) != (T, W) or y.stride(1) != 1:
        raise KernelError("mingru_scan: y must be [T,W]")
    if state.dtype != torch.float32 or state.dim() != 2 or state.shape[1] != W or not state.is_contiguous():
        raise KernelError("mingru_scan: the state is float32 [n_slots, W]")
    _i32(q_start, "q_start")
    _i32(state_slots, "state_slots")
    need = mingru_scan_workspace(n_requests, W, T, max_q_len)
    if need and (workspace is None or workspace.dtype != torch.float32 or workspace.numel() < need):
        raise KernelError(f"mingru_scan: a step with portions of {max_q_len} tokens needs {need} floats of workspace")
    lib = build.load("gated_scan")
    if lib.sglc_gated_scan_chunk() != GATED_SCAN_CHUNK or lib.sglc_gated_scan_piece() != GATED_SCAN_PIECE:
        raise KernelError("gated_scan: the library's chunk size differs from the binding's")
    code = lib.sglc_mingru_scan(_ptr(gate), _ptr(cand), _ptr(out_gate), ctypes.c_longlong(gate.stride(0)), _ptr(y),
                                ctypes.c_longlong(y.stride(0)), _dt(y, "scan output"), _ptr(state), state.shape[0],
                                _ptr(q_start), _ptr(state_slots), int(n_requests), W, T, int(max_q_len),
                                _ptr(workspace), _ptr(tc_error_flag(gate.device)), _stream())
    _check(lib, code, f"mingru_scan (width {W})", n_kernels=2 if need else 1)


def depth_mix(x, hist, n_terms, weights):
    """hist[n_terms-1] = x; x = sum_j weights[j] * hist[j], j < n_terms (32-bit).  x: float32
    [T,E] contiguous; hist: float32 [>= n_terms, T, E] contiguous.  n_terms = 1: only the copy."""
    _need_cuda(x, hist, weights)
    if x.dtype != torch.float32 or hist.dtype != torch.float32 or not x.is_contiguous() or not hist.is_contiguous() \
            or hist.shape[0] < n_terms or tuple(hist.shape[1:]) != tuple(x.shape):
        raise KernelError("depth_mix: x float32 [T,E], hist float32 [n,T,E] with n >= n_terms")
    if n_terms > 1 and (weights is None or weights.dtype != torch.float32 or weights.numel() < n_terms):
        raise KernelError("depth_mix: one float32 weight per term")
    lib = build.load("elementwise")
    code = lib.sglc_depth_mix(_ptr(x), _ptr(hist), ctypes.c_longlong(x.numel()), int(n_terms), _ptr(weights), _stream())
    _check(lib, code, "depth_mix")


def xielu(src, dst, ap, an):
    """dst = xIELU(src): ap*x^2 + x/2 for x > 0, an*(exp(x)-1-x) + x/2 otherwise."""
    _need_cuda(src, dst)
    rows, cols = src.shape
    if tuple(dst.shape) != (rows, cols) or src.stride(1) != 1 or dst.stride(1) != 1:
        raise KernelError("xielu: source and destination must be [rows, cols]")
    lib = build.load("elementwise")
    code = lib.sglc_xielu(_ptr(src), ctypes.c_longlong(src.stride(0)), _dt(src, "xielu source"), _ptr(dst),
                          ctypes.c_longlong(dst.stride(0)), _dt(dst, "xielu destination"), rows, cols,
                          ctypes.c_float(ap), ctypes.c_float(an), _stream())
    _check(lib, code, "xielu")


def set_pdl(on):
    """Turn programmatic dependent launch on or off in every kernel library (on by default)."""
    for name in build.sources():
        build.load(name).sglc_set_pdl(1 if on else 0)


def set_kernel_choice(*, talk_key_split=None):
    """Tuning and test hook.  talk_key_split (on by default): talk_attention_tiles divides a tile's
    keys over a cluster of blocks where the grid is small (off: always one block a tile of queries)."""
    if talk_key_split is not None:
        build.load("attention_talk").sglc_talk_tiles_set_split(1 if talk_key_split else 0)


# ---------------------------------------------------------------------------
# recurrent mixers with a matrix state, their input and output stages
def _f32_rows(t, what, cols=None):
    if t.dtype != torch.float32 or t.dim() != 2 or t.stride(1) != 1 or (cols is not None and t.shape[1] != cols):
        raise KernelError(f"{what} must be float32 rows" + (f" of {cols} columns" if cols is not None else ""))


def short_conv(x, taps, tail, y, token_req, q_start, state_slots, n_requests, segments, unit_eps=1e-6,
               gates=None):
    """Causal convolution over time per channel, silu, and per segment an optional unit-vector
    scaling of each head row (see short_conv.cu).  x: float32 [T, >= C] (the channels are its
    first C columns); taps: float32 [C, K]; tail: float32 [n_slots, K-1, C], a request's last
    K-1 inputs, read and moved on in place; y: float32 [T, C].  segments: (first channel, head
    rows, row width, unit, scale) each, covering the C channels.  gates = (heads, beta column,
    a column, A_log, dt_bias, out [T, 2*heads]): beta = sigmoid(x_b) and decay =
    exp(-exp(A_log) softplus(x_a + dt_bias)) per head, from two more column blocks of x."""
    _need_cuda(x, taps, tail, y, token_req, q_start, state_slots)
    T = y.shape[0]
    C, K = taps.shape
    _f32_rows(x, "short_conv: x")
    _f32_rows(y, "short_conv: y", C)
    if taps.dtype != torch.float32 or not taps.is_contiguous() or x.shape[0] < T or x.shape[1] < C:
        raise KernelError("short_conv: taps float32 [C, K]; x has at least C columns")
    if tail.dtype != torch.float32 or not tail.is_contiguous() or tuple(tail.shape[1:]) != (max(K - 1, 0), C):
        raise KernelError(f"short_conv: the tail is float32 [n_slots, {K - 1}, {C}]")
    for t, nm in ((token_req, "token_req"), (q_start, "q_start"), (state_slots, "state_slots")):
        _i32(t, nm)
    if sum(s[1] * s[2] for s in segments) != C:
        raise KernelError("short_conv: the segments must cover the channels")
    segs = (ctypes.c_int * (4 * len(segments)))(*[int(v) for s in segments for v in s[:4]])
    scales = (ctypes.c_float * len(segments))(*[float(s[4]) for s in segments])
    if gates is not None:
        gh, bcol, acol, a_log, dt_bias, gout = gates
        _need_cuda(a_log, dt_bias, gout)
        _f32_rows(gout, "short_conv: gates", 2 * gh)
        if a_log.dtype != torch.float32 or dt_bias.dtype != torch.float32 or a_log.numel() != gh or dt_bias.numel() != gh \
                or x.shape[1] < max(bcol, acol) + gh:
            raise KernelError("short_conv: A_log and dt_bias are float32 [heads]; x holds both gate column blocks")
    else:
        gh, bcol, acol, a_log, dt_bias, gout = 0, 0, 0, None, None, None
    lib = build.load("short_conv")
    code = lib.sglc_short_conv(_ptr(x), ctypes.c_longlong(x.stride(0)), _ptr(taps), _ptr(tail), _ptr(y),
                               ctypes.c_longlong(y.stride(0)), _ptr(token_req), _ptr(q_start), _ptr(state_slots),
                               T, int(n_requests), C, K, tail.shape[0], ctypes.c_float(unit_eps), segs, scales,
                               len(segments), gh, int(bcol), int(acol), _ptr(a_log), _ptr(dt_bias), _ptr(gout),
                               ctypes.c_longlong(gout.stride(0) if gout is not None else 0),
                               _ptr(tc_error_flag(x.device)), _stream())
    _check(lib, code, f"short_conv (channels {C}, taps {K})", n_kernels=2 if K > 1 and T != int(n_requests) else 1)


MATRIX_STATE_MAX_DIM = 256


def matrix_state(mode, q, k, v, out, state, q_start, state_slots, n_requests, n_heads, n_qk_heads, dim, v_dim,
                 gates=None, head_decay=None, silu_in=False, lower=None, row_z=None, tau=1.0, q_scale=1.0,
                 ones_col=False):
    """A recurrence with a matrix state per head over the step's tokens (see matrix_state.cu).
    mode "decay": S <- d_h S + k v^T (head_decay float32 [H]); mode "delta": the gated delta rule
    (gates float32 [T, 2H]: beta, then decay); mode "row_gate": S <- diag(f) S + (1 - f) v^T with
    f = lower + (1 - lower) sigmoid(k) per head and row (k holds the gates' pre-activations, lower
    float32 [H*dim]; silu_in then acts on q only); mode "row_decay": S <- diag(a) S + k v^T with
    a = sigmoid(row_z)^(1/tau) per head and row (row_z float32 [T, n_qk_heads*dim]); mode "gated":
    S <- g S + b k v^T (gates float32 [T, 2H]: b, then g); with ones_col the state (and out) have
    v_dim columns a head of which the last takes the value 1 for every token, and v has heads of
    v_dim - 1.  q_scale multiplies q.  o = S^T q after the token's write.  q, k: float32
    [T, n_qk_heads*dim]; v: float32 [T, n_heads*v_dim]; out float32 [T, n_heads*v_dim]; state float32
    [n_slots, n_heads, dim, v_dim], read and written in place for the requests' slots."""
    _need_cuda(q, k, v, out, state, q_start, state_slots, gates, head_decay, lower)
    T = out.shape[0]
    _f32_rows(q, "matrix_state: q", n_qk_heads * dim)
    _f32_rows(k, "matrix_state: k", n_qk_heads * dim)
    _f32_rows(v, "matrix_state: v", n_heads * (v_dim - 1 if ones_col else v_dim))
    _f32_rows(out, "matrix_state: out", n_heads * v_dim)
    if state.dtype != torch.float32 or not state.is_contiguous() or tuple(state.shape[1:]) != (n_heads, dim, v_dim):
        raise KernelError(f"matrix_state: the state is float32 [n_slots, {n_heads}, {dim}, {v_dim}]")
    if dim > MATRIX_STATE_MAX_DIM:
        raise KernelError(f"matrix_state: key size {dim} is beyond the kernel's {MATRIX_STATE_MAX_DIM}")
    _i32(q_start, "q_start")
    _i32(state_slots, "state_slots")
    m = {"decay": 0, "delta": 1, "row_gate": 2, "row_decay": 3, "gated": 4}[mode]
    if ones_col and m != 4:
        raise KernelError("matrix_state: the column of ones goes with the gated form")
    if m == 3:
        if row_z is None:
            raise KernelError("matrix_state: the row-decay form takes the decays' pre-activations")
        _need_cuda(row_z)
        _f32_rows(row_z, "matrix_state: row_z", n_qk_heads * dim)
    if m == 2 and (lower is None or lower.dtype != torch.float32 or lower.numel() != n_heads * dim
                   or not lower.is_contiguous() or n_qk_heads != n_heads):
        raise KernelError("matrix_state: the row-gated form takes one float32 lower bound per head and row, "
                          "and as many gate heads as value heads")
    if m == 0 and (head_decay is None or head_decay.dtype != torch.float32 or head_decay.numel() != n_heads):
        raise KernelError("matrix_state: the decay form takes one float32 decay per head")
    if m in (1, 4):
        if gates is None:
            raise KernelError("matrix_state: the delta rule and the gated form take their gates")
        _f32_rows(gates, "matrix_state: gates", 2 * n_heads)
    lib = build.load("matrix_state")
    code = lib.sglc_matrix_state_gen(m, _ptr(q), ctypes.c_longlong(q.stride(0)), _ptr(k), ctypes.c_longlong(k.stride(0)),
                                 _ptr(v), ctypes.c_longlong(v.stride(0)), _ptr(gates),
                                 ctypes.c_longlong(gates.stride(0) if gates is not None else 0), _ptr(head_decay),
                                 _ptr(lower), _ptr(row_z), ctypes.c_longlong(row_z.stride(0) if row_z is not None else 0),
                                 ctypes.c_float(1.0 / float(tau)), ctypes.c_float(q_scale), 1 if ones_col else 0,
                                 _ptr(out), ctypes.c_longlong(out.stride(0)), _ptr(state), state.shape[0],
                                 _ptr(q_start), _ptr(state_slots), int(n_requests), int(n_heads), int(n_qk_heads),
                                 int(dim), int(v_dim), 1 if silu_in else 0, _ptr(tc_error_flag(q.device)), _stream())
    _check(lib, code, f"matrix_state ({mode}, {dim} x {v_dim})")


def gated_norm(o, gate, gain, y, groups, width, eps, act, o_pitch=None, m_run=None):
    """y = o / sqrt(mean(o^2) + eps) * gain * act(gate) per row of `width` (a token has `groups`
    rows side by side; gain float32 [width] serves them all, or [groups*width] every row its own);
    act "silu" or "sigmoid", or "none" with gate None: the norm alone.  o, gate: float32
    [T, groups*width]; y: float32 or bfloat16.  o_pitch: the rows of a token lie so many columns
    apart in o (default width).  m_run (float32 [T, groups], with o_pitch > width): ahead of the
    norm a row is divided by max(|o[width]|, exp(-m_run)) + 1e-6, o[width] being the column behind it."""
    _need_cuda(o, gate, gain, y, m_run)
    T = y.shape[0]
    o_pitch = width if o_pitch is None else int(o_pitch)
    _f32_rows(o, "gated_norm: o", groups * o_pitch)
    if m_run is not None:
        _f32_rows(m_run, "gated_norm: m_run", groups)
        if o_pitch < width + 1 or m_run.shape[0] < T:
            raise KernelError("gated_norm: the divisor's column lies behind the row")
    if (act == "none") != (gate is None):
        raise KernelError("gated_norm: a gate goes with silu or sigmoid, none with \"none\"")
    if gate is not None:
        _f32_rows(gate, "gated_norm: gate", groups * width)
    if gain.dtype != torch.float32 or gain.numel() not in (width, groups * width) or not gain.is_contiguous():
        raise KernelError("gated_norm: the gain is a float32 vector of the row width (or of all rows of a token)")
    if tuple(y.shape) != (T, groups * width) or y.stride(1) != 1 or o.shape[0] < T \
            or (gate is not None and gate.shape[0] < T):
        raise KernelError("gated_norm: y is [T, groups*width]")
    lib = build.load("gated_norm")
    code = lib.sglc_gated_norm_ext(_ptr(o), ctypes.c_longlong(o.stride(0)), _ptr(gate),
                                   ctypes.c_longlong(gate.stride(0) if gate is not None else 0),
                                   _ptr(gain), _ptr(y), ctypes.c_longlong(y.stride(0)), _dt(y, "gated_norm output"), T,
                                   int(groups), int(width), ctypes.c_float(eps),
                                   {"silu": 0, "sigmoid": 1, "none": 2}[act], o_pitch,
                                   1 if (gain.numel() == groups * width and groups > 1) else 0, _ptr(m_run),
                                   ctypes.c_longlong(m_run.stride(0) if m_run is not None else 0), _stream())
    _check(lib, code, f"gated_norm (width {width})")


def rotary_kv(x, positions, freq, mult, dims, norm_eps, q_out, cache, slots, n_heads, n_kv_heads, dim, v_dim,
              page_size):
    """Turn the queries and keys of float32 rows x [T, H*dim | G*dim | G*v_dim] by their positions
    (freq: float64 [dims/2] turns per position of each pair, cos and sin times mult), divide each
    head by its root mean square when norm_eps is not None, write the queries to q_out [T, H*dim]
    and the keys and values into the cache's pages [n_pages, G*page_size*(dim+v_dim)] at slots."""
    _need_cuda(x, positions, freq, q_out, cache, slots)
    T = q_out.shape[0]
    _f32_rows(x, "rotary_kv: x", (n_heads + n_kv_heads) * dim + n_kv_heads * v_dim)
    _i32(positions, "positions")
    _i32(slots, "slots")
    if freq.dtype != torch.float64 or freq.numel() != dims // 2 or not freq.is_contiguous():
        raise KernelError("rotary_kv: one float64 frequency per turned pair")
    if q_out.shape[1] != n_heads * dim or q_out.stride(1) != 1 or q_out.dtype != cache.dtype or not cache.is_contiguous():
        raise KernelError("rotary_kv: queries [T, H*dim] and the cache have one dtype")
    n_pages = cache.shape[0]
    if cache.numel() != n_pages * n_kv_heads * page_size * (dim + v_dim):
        raise KernelError(f"rotary_kv: cache {tuple(cache.shape)} does not fit {n_kv_heads} heads of {dim}+{v_dim}")
    lib = build.load("rotary")
    code = lib.sglc_rotary_kv(_ptr(x), ctypes.c_longlong(x.stride(0)), _ptr(positions), _ptr(freq), ctypes.c_float(mult),
                              int(dims), 0 if norm_eps is None else 1, ctypes.c_float(norm_eps or 0.0), _ptr(q_out),
                              ctypes.c_longlong(q_out.stride(0)), _ptr(cache), _ptr(slots), T, int(n_heads),
                              int(n_kv_heads), int(dim), int(v_dim), int(page_size), n_pages, _dt(q_out, "queries"),
                              _ptr(tc_error_flag(x.device)), _stream())
    _check(lib, code, f"rotary_kv (head {dim})")


QK_NORMS = {None: 0, False: 0, "none": 0, True: 1, "unit": 1, "head_gain": 2, "row_gain": 3}


def qk_prep(x, positions, freq, mult, dims, pairing, norm, eps, gain_q, gain_k, q_out, cache, slots, n_heads,
            n_kv_heads, dim, v_dim, page_size, v_mult=1.0):
    """The general input stage of a softmax attention (rotary.cu: qk_prep_kernel).  x: float32 rows
    [T, H*dim | G*dim | G*v_dim], or [T, H*dim] alone with n_kv_heads = 0 (a layer that reads keys and
    values another layer cached: cache and slots are then None).  norm: None; "unit" (after the
    turn, no gain); "head_gain" (before the turn, per head, gains float32 [dim] shared by the heads);
    "row_gain" (before the turn, one root mean square over all query heads and one over all key
    heads, gains float32 [H*dim] and [G*dim]).  pairing "halves" or "neighbours".  Queries go to q_out
    [T, H*dim]; keys and values (times v_mult) into the cache's pages at slots."""
    _need_cuda(x, positions, freq, q_out, cache, slots, gain_q, gain_k)
    T = q_out.shape[0]
    G = int(n_kv_heads)
    _f32_rows(x, "qk_prep: x", n_heads * dim + G * (dim + v_dim))
    _i32(positions, "positions")
    mode = QK_NORMS[norm]
    if dims and (freq is None or freq.dtype != torch.float64 or freq.numel() != dims // 2 or not freq.is_contiguous()):
        raise KernelError("qk_prep: one float64 frequency per turned pair")
    if q_out.shape[1] != n_heads * dim or q_out.stride(1) != 1:
        raise KernelError("qk_prep: queries [T, H*dim]")
    n_pages = 0
    if G:
        _i32(slots, "slots")
        n_pages = cache.shape[0]
        if q_out.dtype != cache.dtype or not cache.is_contiguous() \
                or cache.numel() != n_pages * G * page_size * (dim + v_dim):
            raise KernelError(f"qk_prep: cache {tuple(cache.shape)} does not fit {G} heads of {dim}+{v_dim}, or its "
                              "dtype is not the queries'")
    want = {2: (dim, dim if G else 0), 3: (n_heads * dim, G * dim)}.get(mode)
    if want is not None:
        for g, n, nm in ((gain_q, want[0], "queries"), (gain_k, want[1], "keys")):
            if n and (g is None or g.dtype != torch.float32 or g.numel() != n or not g.is_contiguous()):
                raise KernelError(f"qk_prep: the gain of the {nm} is a float32 vector of {n}")
    lib = build.load("rotary")
    code = lib.sglc_qk_prep(_ptr(x), ctypes.c_longlong(x.stride(0)), _ptr(positions), _ptr(freq if dims else None),
                            ctypes.c_float(mult), int(dims), ROTARY_PAIRINGS[pairing], mode, ctypes.c_float(eps or 0.0),
                            _ptr(gain_q), _ptr(gain_k if G else None), ctypes.c_float(v_mult), _ptr(q_out),
                            ctypes.c_longlong(q_out.stride(0)), _ptr(cache if G else None), _ptr(slots if G else None),
                            T, int(n_heads), G, int(dim), int(v_dim), int(page_size), n_pages, _dt(q_out, "queries"),
                            _ptr(tc_error_flag(x.device)), _stream())
    _check(lib, code, f"qk_prep (head {dim})")


def stabilized_gates(xi, xf, cap, gates, m_out, m_state, q_start, state_slots, n_requests, n_heads):
    """Exponential gates with a running maximum per (request, head) (matrix_state.cu:
    stabilized_gates_kernel).  xi, xf: float32 [T, n_heads] views (the input and forget gates'
    pre-activations, biases included); gates: float32 [T, 2*n_heads] (input weight, then decay);
    m_out: float32 [T, n_heads]; m_state: float32 [n_slots, n_heads], read and written in place."""
    _need_cuda(xi, xf, gates, m_out, m_state, q_start, state_slots)
    _f32_rows(xi, "stabilized_gates: xi", n_heads)
    _f32_rows(xf, "stabilized_gates: xf", n_heads)
    _f32_rows(gates, "stabilized_gates: gates", 2 * n_heads)
    _f32_rows(m_out, "stabilized_gates: m_out", n_heads)
    if m_state.dtype != torch.float32 or not m_state.is_contiguous() or tuple(m_state.shape[1:]) != (n_heads,):
        raise KernelError(f"stabilized_gates: the running maxima are float32 [n_slots, {n_heads}]")
    _i32(q_start, "q_start")
    _i32(state_slots, "state_slots")
    lib = build.load("matrix_state")
    code = lib.sglc_stabilized_gates(_ptr(xi), ctypes.c_longlong(xi.stride(0)), _ptr(xf), ctypes.c_longlong(xf.stride(0)),
                                     ctypes.c_float(cap), _ptr(gates), ctypes.c_longlong(gates.stride(0)), _ptr(m_out),
                                     ctypes.c_longlong(m_out.stride(0)), _ptr(m_state), m_state.shape[0], _ptr(q_start),
                                     _ptr(state_slots), int(n_requests), int(n_heads), _ptr(tc_error_flag(xi.device)),
                                     _stream())
    _check(lib, code, f"stabilized_gates ({n_heads} heads)")


def gated_gather(z, tokens, table, first, dst, err_flag=None):
    """dst[t, j] = gelu_tanh(z[t, j]) * table[tokens[t], first + j] for the columns dst has; z float32
    rows; table float32 or bfloat16 [rows, cols]."""
    _need_cuda(z, tokens, table, dst)
    rows, cols = dst.shape
    _f32_rows(z, "gated_gather: z")
    _i32(tokens, "tokens")
    if z.shape[0] < rows or z.shape[1] < cols or dst.stride(1) != 1 or table.dim() != 2 or not table.is_contiguous():
        raise KernelError("gated_gather: z float32 [>= rows, >= cols]; dst rows contiguous; a contiguous table")
    lib = build.load("elementwise")
    code = lib.sglc_gated_gather(_ptr(z), ctypes.c_longlong(z.stride(0)), _ptr(tokens), _ptr(table),
                                 ctypes.c_longlong(table.shape[1]), table.shape[0], int(first), _dt(table, "table"),
                                 _ptr(dst), ctypes.c_longlong(dst.stride(0)), _dt(dst, "gated_gather destination"),
                                 rows, cols, _ptr(err_flag), _stream())
    _check(lib, code, "gated_gather")


EXT_MAX_SPLITS = 16         # blocks a token's keys are dealt to at most (attention_ext in a step of single tokens)


def attention_ext_splits(max_keys, window=None, chunk=None):
    """How many blocks share a token's keys in a step of single tokens: two tiles of 32 keys a block,
    up to EXT_MAX_SPLITS (1: the plain launch)."""
    seen = min(int(max_keys), int(window or max_keys), int(chunk or max_keys))
    tiles = (seen + 31) // 32 + 1
    return max(1, min(EXT_MAX_SPLITS, tiles // 2))


def attention_ext(q, cache, block_table, token_req, positions, out, n_heads, n_kv_heads, dim, v_dim, page_size,
                  scale, window, chunk, sinks, max_keys, max_q_len=None, splits=1, workspace=None):
    """attention_simt's extended form: values of size v_dim beside keys of size dim (cache
    [n_pages, G*page_size*(dim+v_dim)]: a page's keys, then its values), an optional chunk mask
    (a query sees the keys of its own chunk of `chunk` positions) and an optional sink per head
    (float32 [H]) in the softmax's denominator.  q [T, H*dim]; out [T, H*v_dim].
    splits > 1 (a step of single tokens only): every token's keys are dealt to so many blocks, whose
    shares a second launch merges; workspace: float32, T * H * splits * (v_dim + 2) entries."""
    _need_cuda(q, cache, block_table, token_req, positions, out, sinks, workspace)
    for t, nm in ((block_table, "block_table"), (token_req, "token_req"), (positions, "positions")):
        _i32(t, nm)
    T = q.shape[0]
    n_pages = cache.shape[0]
    if q.shape[1] != n_heads * dim or out.shape[1] != n_heads * v_dim or q.stride(1) != 1 or out.stride(1) != 1 \
            or q.dtype != out.dtype or q.dtype != cache.dtype or not cache.is_contiguous():
        raise KernelError("attention_ext: q [T, H*dim], out [T, H*v_dim] and the cache have one dtype")
    if cache.numel() != n_pages * n_kv_heads * page_size * (dim + v_dim):
        raise KernelError(f"attention_ext: cache {tuple(cache.shape)} does not fit {n_kv_heads} heads of {dim}+{v_dim}")
    if sinks is not None and (sinks.dtype != torch.float32 or sinks.numel() != n_heads):
        raise KernelError("attention_ext: one float32 sink per head")
    lib = build.load("attention_simt")
    if splits > 1:
        if (max_q_len or 2) > 1 or workspace is None or workspace.dtype != torch.float32 \
                or workspace.numel() < T * n_heads * splits * (v_dim + 2) or not workspace.is_contiguous():
            raise KernelError("attention_ext: keys are split over blocks in a step of single tokens only, with a "
                              "float32 workspace of T * H * splits * (v_dim + 2) entries")
        code = lib.sglc_attention_simt_ext_split(
            _ptr(q), q.stride(0), _ptr(cache), _ptr(block_table), block_table.stride(0), _ptr(token_req),
            _ptr(positions), _ptr(out), out.stride(0), T, int(n_heads), int(n_kv_heads), int(dim), int(v_dim),
            int(page_size), ctypes.c_float(scale), int(window or 0), int(chunk or 0), _ptr(sinks), int(max_keys),
            _dt(q, "attention q"), _dt(cache, "cache"), n_pages, _ptr(tc_error_flag(q.device)), int(splits),
            _ptr(workspace), _stream())
        _check(lib, code, f"attention_ext (head {dim}/{v_dim}, up to {max_keys} keys, {splits} shares)", n_kernels=2)
        return
    code = lib.sglc_attention_simt_ext(_ptr(q), q.stride(0), _ptr(cache), _ptr(block_table), block_table.stride(0),
                                       _ptr(token_req), _ptr(positions), _ptr(out), out.stride(0), T, int(n_heads),
                                       int(n_kv_heads), int(dim), int(v_dim), int(page_size), ctypes.c_float(scale),
                                       int(window or 0), int(chunk or 0), _ptr(sinks), int(max_keys),
                                       _dt(q, "attention q"), _dt(cache, "cache"), n_pages,
                                       _ptr(tc_error_flag(q.device)), int(max_q_len) if max_q_len else 2, _stream())
    _check(lib, code, f"attention_ext (head {dim}/{v_dim}, up to {max_keys} keys)")


GATE_ACTS = {"silu": 0, "gelu_tanh": 1}


def gated_act(src, dst, weights=None, per=0, act="silu", mult=1.0, n_weighted=None):
    """dst[r, j] = act(src[r, j]) * src[r, F + j] (* weights[r, j // per]) * mult; src [rows, 2F] holds
    the gate columns, then the up columns; weights: float32 [rows, F // per] or None; act "silu" or
    "gelu_tanh"; mult: one more factor of every result, taken in 32-bit.  n_weighted: only the
    first so many columns (a multiple of per) take weights, [rows, n_weighted // per]; the rest take 1."""
    _need_cuda(src, dst, weights)
    rows, F = dst.shape
    if src.shape[1] != 2 * F or src.shape[0] < rows or src.stride(1) != 1 or dst.stride(1) != 1:
        raise KernelError("gated_act: src [rows, 2F], dst [rows, F]")
    if weights is not None:
        _f32_rows(weights, "gated_act: weights")
        nw = F if n_weighted is None else int(n_weighted)
        if per <= 0 or nw % per or nw > F or weights.shape[1] != nw // per or weights.shape[0] < rows:
            raise KernelError("gated_act: one weight per row and block of `per` columns")
    else:
        nw = F
    lib = build.load("elementwise")
    code = lib.sglc_gated_act_part(_ptr(src), ctypes.c_longlong(src.stride(0)), _dt(src, "gated_act source"), _ptr(dst),
                                   ctypes.c_longlong(dst.stride(0)), _dt(dst, "gated_act destination"), rows, F,
                                   _ptr(weights), ctypes.c_longlong(weights.stride(0) if weights is not None else 0),
                                   int(per), GATE_ACTS[act], ctypes.c_float(mult), nw, _stream())
    _check(lib, code, "gated_act")


ROUTER_MAX_EXPERTS = 256


def router(logits, correction, dense, ids, weights, top, n_groups=1, keep=1, renorm=False, weight_scale=1.0,
           score="sigmoid", renorm_eps=0.0):
    """Routing by sigmoid scores (or, score "softmax", a softmax over all experts) with a choice
    correction and group limits; renorm: the chosen scores divided by their sum + renorm_eps; then
    times weight_scale (see router.cu).  logits: float32
    [T, E]; correction: float32 [E] or None; dense: float32 [T, E] (weights, zero where not
    chosen); ids int32 [T, top]; weights float32 [T, top]."""
    _need_cuda(logits, correction, dense, ids, weights)
    T, E = dense.shape
    _f32_rows(logits, "router: logits", E)
    _f32_rows(dense, "router: dense", E)
    if ids.dtype != torch.int32 or not ids.is_contiguous() or tuple(ids.shape) != (T, top) \
            or weights.dtype != torch.float32 or not weights.is_contiguous() or tuple(weights.shape) != (T, top):
        raise KernelError("router: ids int32 [T, top], weights float32 [T, top]")
    if correction is not None and (correction.dtype != torch.float32 or correction.numel() != E):
        raise KernelError("router: one float32 correction per expert")
    lib = build.load("router")
    code = lib.sglc_router_ext(_ptr(logits), ctypes.c_longlong(logits.stride(0)), _ptr(correction), _ptr(dense),
                               ctypes.c_longlong(dense.stride(0)), _ptr(ids), _ptr(weights), T, E, int(top),
                               int(n_groups), int(keep), 1 if renorm else 0, ctypes.c_float(weight_scale),
                               {"sigmoid": 0, "softmax": 1}[score], ctypes.c_float(renorm_eps), _stream())
    _check(lib, code, f"router ({E} experts, {top} chosen)")


def cast_rows(src, dst):
    """dst[r, j] = src[r, j] for the columns dst has: float32 rows into rows (a column range of
    wider rows, if dst is such a view) of float32 or bfloat16."""
    _need_cuda(src, dst)
    rows, cols = dst.shape
    _f32_rows(src, "cast_rows: src")
    if src.shape[0] < rows or src.shape[1] < cols or dst.stride(1) != 1:
        raise KernelError("cast_rows: src float32 [>= rows, >= cols]; dst rows contiguous")
    lib = build.load("elementwise")
    code = lib.sglc_cast_rows(_ptr(src), ctypes.c_longlong(src.stride(0)), _ptr(dst), ctypes.c_longlong(dst.stride(0)),
                              _dt(dst, "cast_rows destination"), rows, cols, _stream())
    _check(lib, code, "cast_rows")


ROTARY_PAIRINGS = {"halves": 0, "neighbours": 1}


def latent_rope(qx, low, gain, eps, positions, freq, mult, dims, pairing, q_out, rows, slots, n_heads, rank, rot_dim):
    """The input stage of a latent attention with a turned part (see rotary.cu).  qx: float32
    [T, H*(rank+rot_dim)], every head [rank entries that pass | rot_dim entries turned by position];
    low: float32 [T, rank+rot_dim] or None, the token's latent (its first `rank` entries divided by
    their root mean square, times gain) and one shared key part (turned), written to `rows`
    [n_rows, rank+rot_dim] at slots; q_out [T, H*(rank+rot_dim)] in the cache's precision.  Of the
    rot_dim entries the first `dims` are turned: pairs (i, i + dims/2) ("halves") or (2i, 2i+1)
    ("neighbours"); freq float64 [dims/2]."""
    _need_cuda(qx, low, gain, positions, freq, q_out, rows, slots)
    T = q_out.shape[0]
    W = rank + rot_dim
    _f32_rows(qx, "latent_rope: qx", n_heads * W)
    _i32(positions, "positions")
    if freq.dtype != torch.float64 or freq.numel() != dims // 2 or not freq.is_contiguous():
        raise KernelError("latent_rope: one float64 frequency per turned pair")
    if tuple(q_out.shape) != (T, n_heads * W) or q_out.stride(1) != 1:
        raise KernelError("latent_rope: queries leave as [T, heads*(rank+rot_dim)]")
    n_rows = 0
    if low is not None:
        _f32_rows(low, "latent_rope: low", W)
        _i32(slots, "slots")
        if gain.dtype != torch.float32 or gain.numel() != rank or rows.dim() != 2 or rows.shape[1] != W \
                or not rows.is_contiguous() or rows.dtype != q_out.dtype:
            raise KernelError("latent_rope: gain float32 [rank]; cache rows [n, rank+rot_dim] of the queries' dtype")
        n_rows = rows.shape[0]
    lib = build.load("rotary")
    code = lib.sglc_latent_rope(_ptr(qx), ctypes.c_longlong(qx.stride(0)), _ptr(low),
                                ctypes.c_longlong(low.stride(0) if low is not None else 0), _ptr(gain),
                                ctypes.c_float(eps), _ptr(positions), _ptr(freq), ctypes.c_float(mult), int(dims),
                                ROTARY_PAIRINGS[pairing], _ptr(q_out), ctypes.c_longlong(q_out.stride(0)),
                                _ptr(rows if low is not None else None), _ptr(slots if low is not None else None),
                                ctypes.c_longlong(n_rows), T, int(n_heads), int(rank), int(rot_dim),
                                _dt(q_out, "latent_rope queries"), _ptr(tc_error_flag(qx.device)), _stream())
    _check(lib, code, f"latent_rope (rank {rank}, turned {rot_dim})")


TALK_MAX_HEADS, TALK_MAX_DIM = 32, 256


def talk_prep(x, wq, wk, eps, q_out, cache, slots, n_heads, n_kv_heads, dim, page_size):
    """The input stage of a talking-heads attention (see attention_talk.cu).  x: float32 [T, >=
    (H+G)*dim], queries then keys as projected; wq, wk: float32 [dim], the gains of the queries'
    and keys' norms; q_out: float32 [T, H*dim], the normalised queries times both gains; the keys
    go as they are into cache [n_pages, 1, G, page_size, dim] at slots."""
    _need_cuda(x, wq, wk, q_out, cache, slots)
    T = q_out.shape[0]
    _f32_rows(x, "talk_prep: x")
    _f32_rows(q_out, "talk_prep: q_out", n_heads * dim)
    _i32(slots, "slots")
    n_pages = cache.shape[0]
    if x.shape[1] < (n_heads + n_kv_heads) * dim or x.shape[0] < T or not cache.is_contiguous() \
            or cache.numel() != n_pages * n_kv_heads * page_size * dim:
        raise KernelError(f"talk_prep: x holds queries and keys; cache {tuple(cache.shape)} keeps one row per "
                          f"position and each of {n_kv_heads} heads of {dim}")
    for v in (wq, wk):
        if v.dtype != torch.float32 or v.numel() != dim or not v.is_contiguous():
            raise KernelError("talk_prep: the norms' gains are float32 [dim]")
    lib = build.load("attention_talk")
    code = lib.sglc_talk_prep(_ptr(x), ctypes.c_longlong(x.stride(0)), _ptr(wq), _ptr(wk), ctypes.c_float(eps),
                              _ptr(q_out), ctypes.c_longlong(q_out.stride(0)), _ptr(cache), _dt(cache, "cache"),
                              _ptr(slots), T, int(n_heads), int(n_kv_heads), int(dim), int(page_size), n_pages,
                              _ptr(tc_error_flag(x.device)), _stream())
    _check(lib, code, f"talk_prep (head {dim})")


def talk_attention(q, cache, block_table, token_req, positions, slopes, talk, gate, out, n_heads, n_kv_heads, dim,
                   page_size, scale, eps, mult, window):
    """Softmax attention with a distance penalty per head, the heads' weights mixed after the
    softmax, values that are the cached keys, and a sigmoid output gate (see attention_talk.cu).
    q: float32 [T, H*dim] from talk_prep; slopes float32 [H]; talk float32 [H, H]; gate: float32
    rows [T, H*dim] or None; out [T, H*dim] of the cache's dtype; token_req None: token t is the
    step's t-th request."""
    _need_cuda(q, cache, block_table, token_req, positions, slopes, talk, gate, out)
    T = out.shape[0]
    _f32_rows(q, "talk_attention: q", n_heads * dim)
    for t, nm in ((block_table, "block_table"), (positions, "positions")):
        _i32(t, nm)
    if token_req is not None:
        _i32(token_req, "token_req")
    if gate is not None:
        _f32_rows(gate, "talk_attention: gate", n_heads * dim)
    n_pages = cache.shape[0]
    if slopes.dtype != torch.float32 or slopes.numel() != n_heads or talk.dtype != torch.float32 \
            or talk.numel() != n_heads * n_heads or not talk.is_contiguous():
        raise KernelError("talk_attention: slopes float32 [H], talk float32 [H, H]")
    if tuple(out.shape) != (T, n_heads * dim) or out.stride(1) != 1 or out.dtype != cache.dtype \
            or not cache.is_contiguous() or cache.numel() != n_pages * n_kv_heads * page_size * dim:
        raise KernelError("talk_attention: out [T, H*dim] and the cache have one dtype")
    if n_heads > TALK_MAX_HEADS or dim > TALK_MAX_DIM:
        raise KernelError(f"talk_attention: up to {TALK_MAX_HEADS} heads of up to {TALK_MAX_DIM}")
    lib = build.load("attention_talk")
    code = lib.sglc_talk_attention(_ptr(q), ctypes.c_longlong(q.stride(0)), _ptr(cache), _dt(cache, "cache"),
                                   _ptr(block_table), block_table.stride(0), _ptr(token_req), _ptr(positions),
                                   _ptr(slopes), _ptr(talk), _ptr(gate),
                                   ctypes.c_longlong(gate.stride(0) if gate is not None else 0), _ptr(out),
                                   ctypes.c_longlong(out.stride(0)), _dt(out, "talk_attention output"), T,
                                   int(n_heads), int(n_kv_heads), int(dim), int(page_size), ctypes.c_float(scale),
                                   ctypes.c_float(eps), ctypes.c_float(mult), int(window or 0), n_pages,
                                   _ptr(tc_error_flag(q.device)), _stream())
    _check(lib, code, f"talk_attention (head {dim}, {n_heads} heads)")


TALK_TILES_MAX_HEADS = 16
_TALK_UNSUPPORTED = -2


def talk_attention_tiles(q, cache, block_table, q_start, kv_len, slopes, talk, gate, out, n_requests, max_q_len,
                         n_heads, n_kv_heads, dim, page_size, scale, eps, mult, window, max_keys=0):
    """talk_attention in tiles of 16 queries on the tensor cores, for a bfloat16 cache and output
    (see attention_talk.cu): the step's requests r bring tokens q_start[r] .. q_start[r+1]-1 and
    hold kv_len[r] positions after it (max_keys: a bound on those, or 0; it only sizes the staging:
    where a block's whole key range fits its shared memory, every key is fetched once).  Returns False, having launched nothing, where the sizes
    have no tiled form (head size not 32/48/64/96/128, more than 16 heads, too much shared memory,
    rows not aligned): the caller then takes talk_attention."""
    if cache.dtype != torch.bfloat16 or out.dtype != torch.bfloat16 or n_heads > TALK_TILES_MAX_HEADS \
            or dim not in (32, 48, 64, 96, 128):
        return False
    _need_cuda(q, cache, block_table, q_start, kv_len, slopes, talk, gate, out)
    _f32_rows(q, "talk_attention_tiles: q", n_heads * dim)
    for t, nm in ((block_table, "block_table"), (q_start, "q_start"), (kv_len, "kv_len")):
        _i32(t, nm)
    if gate is not None:
        _f32_rows(gate, "talk_attention_tiles: gate", n_heads * dim)
    n_pages = cache.shape[0]
    if slopes.dtype != torch.float32 or slopes.numel() != n_heads or talk.dtype != torch.float32 \
            or talk.numel() != n_heads * n_heads or not talk.is_contiguous():
        raise KernelError("talk_attention_tiles: slopes float32 [H], talk float32 [H, H]")
    if out.shape[1] != n_heads * dim or out.stride(1) != 1 or not cache.is_contiguous() \
            or cache.numel() != n_pages * n_kv_heads * page_size * dim:
        raise KernelError("talk_attention_tiles: out [T, H*dim]; the cache keeps one row per position and key head")
    lib = build.load("attention_talk")
    code = lib.sglc_talk_attention_tiles(
        _ptr(q), ctypes.c_longlong(q.stride(0)), _ptr(cache), _ptr(block_table), block_table.stride(0), _ptr(q_start),
        _ptr(kv_len), _ptr(slopes), _ptr(talk), _ptr(gate), ctypes.c_longlong(gate.stride(0) if gate is not None else 0),
        _ptr(out), ctypes.c_longlong(out.stride(0)), int(n_requests), int(max_q_len), int(max_keys or 0), int(n_heads),
        int(n_kv_heads),
        int(dim), int(page_size), ctypes.c_float(scale), ctypes.c_float(eps), ctypes.c_float(mult), int(window or 0),
        n_pages, _ptr(tc_error_flag(q.device)), _stream())
    if code == _TALK_UNSUPPORTED:
        return False
    _check(lib, code, f"talk_attention_tiles (head {dim}, {n_heads} heads)")
    return True
