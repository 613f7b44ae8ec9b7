"""Host side of tensor parallelism on CPU: the shard cutter is checked bit-exactly against slices of
the dequantised matrix, and a two-process gloo run checks that the collective placement (one
all-reduce after wo, one after w2, an all-gather of the vocabulary shards' best tokens) reproduces
the single-process forward pass."""
import os
import socket
import tempfile

import numpy as np
import pytest

import jitllm_b200 as jl
from jitllm_b200.tensor_parallel import check_divisible

from tests.np_formats import DEQUANT
from tests.np_forward import NpLlama, matvec, rmsnorm, seq_sum

F = np.float32
CFG = jl.Configuration(dim=512, hiddenDim=1024, numberOfLayers=2, numberOfHeads=4, numberOfKeyValueHeads=2,
                       vocabularySize=512, contextLength=8)
SEED = 4242


@pytest.mark.parametrize("fmt", [jl.GGMLType.Q8_0, jl.GGMLType.Q4_0, jl.GGMLType.Q4_K])
@pytest.mark.parametrize("size", [2, 4])
def test_shards_are_slices_of_the_matrix(fmt, size):
    cfg = jl.Configuration(dim=1024, hiddenDim=2048, numberOfLayers=1, numberOfHeads=8, numberOfKeyValueHeads=4,
                           vocabularySize=256, contextLength=8)
    for role in (jl.TensorRole.ATTENTION_QUERY, jl.TensorRole.ATTENTION_KEY, jl.TensorRole.FFN_UP,
                 jl.TensorRole.OUTPUT, jl.TensorRole.ATTENTION_OUTPUT, jl.TensorRole.FFN_DOWN):
        rows, cols = cfg.matrix_shape(role)
        raw = jl.synth_tensor(fmt, rows * cols, 17 + int(role))
        full = DEQUANT[int(fmt)](raw).reshape(rows, cols)
        seen = []
        for rank in range(size):
            tp = jl.TensorParallel(rank, size)
            lr, lc = jl.local_shape(cfg, role, size)
            part = jl.shard_tensor(cfg, role, fmt, raw, tp)
            assert part.nbytes == fmt.byte_size_for(lr * lc)
            got = DEQUANT[int(fmt)](part).reshape(lr, lc)
            if lr != rows:
                want = full[rank * lr:(rank + 1) * lr]
            else:
                want = full[:, rank * lc:(rank + 1) * lc]
            assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
            seen.append(got)
        axis = 0 if seen[0].shape[0] != rows else 1
        assert np.array_equal(np.concatenate(seen, axis=axis), full)


def test_replicated_roles_are_untouched():
    raw = np.arange(CFG.dim, dtype=np.float32)
    tp = jl.TensorParallel(1, 2)
    assert jl.shard_tensor(CFG, jl.TensorRole.ATTENTION_NORM, jl.GGMLType.F32, raw, tp) is raw
    assert jl.local_shape(CFG, jl.TensorRole.TOKEN_EMBEDDING, 2) == (CFG.vocabularySize, CFG.dim)


def test_bad_splits_are_rejected_on_the_host():
    with pytest.raises(ValueError, match="GPUL-CFG-002"):
        check_divisible(CFG, 3)
    with pytest.raises(ValueError, match="GPUL-CFG-002"):
        check_divisible(CFG, 4)  # 512 / 4 = 128 columns per GPU: not a whole 256-group
    with pytest.raises(ValueError, match="GPUL-CFG-002"):
        jl.TensorParallel(2, 2)
    check_divisible(CFG, 2)


def _weights(tensors, cfg, tp):
    """Dequantised local shards in the layout NpLlama uses."""
    def m(role, layer):
        t, raw = tensors[(role, layer)]
        return DEQUANT[int(t)](jl.shard_tensor(cfg, role, t, raw, tp))
    R = jl.TensorRole
    L = range(cfg.numberOfLayers)
    cr, ci = jl.precomputeFreqsCis(cfg.contextLength, cfg.headSize, cfg.ropeTheta)
    return {
        "emb": m(R.TOKEN_EMBEDDING, -1), "wcls": m(R.OUTPUT, -1), "final_norm": tensors[(R.OUTPUT_NORM, -1)][1],
        "att_norm": [tensors[(R.ATTENTION_NORM, l)][1] for l in L], "ffn_norm": [tensors[(R.FFN_NORM, l)][1] for l in L],
        "wq": [m(R.ATTENTION_QUERY, l) for l in L], "wk": [m(R.ATTENTION_KEY, l) for l in L],
        "wv": [m(R.ATTENTION_VALUE, l) for l in L], "wo": [m(R.ATTENTION_OUTPUT, l) for l in L],
        "w1": [m(R.FFN_GATE, l) for l in L], "w3": [m(R.FFN_UP, l) for l in L], "w2": [m(R.FFN_DOWN, l) for l in L],
        "cr": cr, "ci": ci,
    }


def _np_cfg(cfg):
    return {"dim": cfg.dim, "head": cfg.headSize, "kv_dim": cfg.kvDim, "heads": cfg.numberOfHeads,
            "kv_heads": cfg.numberOfKeyValueHeads, "layers": cfg.numberOfLayers, "ctx": cfg.contextLength,
            "hidden": cfg.hiddenDim, "vocab": cfg.vocabularySize, "eps": cfg.rmsNormEps}


def _tp_forward(cfg, w, tp, kc, vc, token, pos, all_reduce, all_gather):
    """One rank's share of the forward pass: local heads, local hidden columns, local vocabulary rows;
    `all_reduce` where the library calls NCCL."""
    dim, hs = cfg.dim, cfg.headSize
    heads, kvh = cfg.numberOfHeads // tp.size, cfg.numberOfKeyValueHeads // tp.size
    qdim, kvd, hid, voc = heads * hs, kvh * hs, cfg.hiddenDim // tp.size, cfg.vocabularySize // tp.size
    x = w["emb"][token * dim:(token + 1) * dim].copy()
    for l in range(cfg.numberOfLayers):
        xb = rmsnorm(x, w["att_norm"][l], cfg.rmsNormEps)
        q, k, v = matvec(w["wq"][l], xb, qdim, dim), matvec(w["wk"][l], xb, kvd, dim), matvec(w["wv"][l], xb, kvd, dim)
        for vec in (q, k):
            for i in range(0, vec.size, 2):
                fcr, fci = w["cr"][pos * (hs // 2) + (i % hs) // 2], w["ci"][pos * (hs // 2) + (i % hs) // 2]
                v0, v1 = vec[i], vec[i + 1]
                vec[i], vec[i + 1] = F(F(v0 * fcr) - F(v1 * fci)), F(F(v0 * fci) + F(v1 * fcr))
        kc[l, pos], vc[l, pos] = k.astype(np.float16), v.astype(np.float16)
        out = np.zeros(qdim, dtype=F)
        for h in range(heads):
            g = h // (heads // kvh)
            kh, vh = kc[l, :pos + 1, g * hs:(g + 1) * hs].astype(F), vc[l, :pos + 1, g * hs:(g + 1) * hs].astype(F)
            sc = np.cumsum((q[None, h * hs:(h + 1) * hs] * kh).astype(F), axis=1, dtype=F)[:, -1]
            sc = (sc / F(np.sqrt(np.float64(hs)))).astype(F)
            e = np.exp((sc - sc.max()).astype(F).astype(np.float64)).astype(F)
            a = (e / seq_sum(e)).astype(F)
            acc = np.zeros(hs, dtype=F)
            for t in range(pos + 1):
                acc = ((a[t] * vh[t]).astype(F) + acc).astype(F)
            out[h * hs:(h + 1) * hs] = acc
        x = (x + all_reduce(matvec(w["wo"][l], out, dim, qdim))).astype(F)
        xb = rmsnorm(x, w["ffn_norm"][l], cfg.rmsNormEps)
        g, u = matvec(w["w1"][l], xb, hid, dim), matvec(w["w3"][l], xb, hid, dim)
        g = (g / (1.0 + np.exp(-g.astype(np.float64))).astype(F)).astype(F)
        x = (x + all_reduce(matvec(w["w2"][l], (g * u).astype(F), dim, hid))).astype(F)
    logits = matvec(w["wcls"], rmsnorm(x, w["final_norm"], cfg.rmsNormEps), voc, dim)
    best = int(np.argmax(logits))  # first maximum
    pairs = all_gather(np.array([logits[best], best + tp.rank * voc], dtype=np.float64))
    k = max(range(tp.size), key=lambda r: (pairs[r][0], -pairs[r][1]))
    return logits, int(pairs[k][1])


def _rank_main(rank, size, port, out_dir):
    import torch
    import torch.distributed as dist
    torch.set_num_threads(1)
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=size)
    try:
        tp = jl.TensorParallel(rank, size)
        tensors = jl.synth_model_tensors(CFG, jl.GGMLType.Q4_K, SEED, std=0.05)
        w = _weights(tensors, CFG, tp)
        kc = np.zeros((CFG.numberOfLayers, CFG.contextLength, CFG.kvDim // size), dtype=np.float16)
        vc = np.zeros_like(kc)

        def all_reduce(a):
            t = torch.from_numpy(np.ascontiguousarray(a))
            dist.all_reduce(t)
            return t.numpy()

        def all_gather(a):
            parts = [torch.zeros(a.size, dtype=torch.float64) for _ in range(size)]
            dist.all_gather(parts, torch.from_numpy(a))
            return [p.numpy() for p in parts]

        # the id channel init_group uses, exercised without a GPU
        payload = jl.torch_broadcast(bytes(range(128)) if rank == 0 else None)
        assert payload == bytes(range(128))
        toks, rows = [], []
        token = 7
        for pos in range(3):
            logits, token = _tp_forward(CFG, w, tp, kc, vc, token, pos, all_reduce, all_gather)
            toks.append(token)
            rows.append(logits)
        np.savez(os.path.join(out_dir, f"rank{rank}.npz"), tokens=np.array(toks), logits=np.stack(rows))
    finally:
        dist.destroy_process_group()


def test_two_ranks_over_gloo_match_one_rank():
    import torch.multiprocessing as mp
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    size = 2
    with tempfile.TemporaryDirectory() as d:
        mp.spawn(_rank_main, args=(size, port, d), nprocs=size, join=True)
        got = [np.load(os.path.join(d, f"rank{r}.npz")) for r in range(size)]
    tensors = jl.synth_model_tensors(CFG, jl.GGMLType.Q4_K, SEED, std=0.05)
    ref = NpLlama(_np_cfg(CFG), _weights(tensors, CFG, jl.TensorParallel()))
    token = 7
    for pos in range(3):
        want = ref.forward(token, pos)
        have = np.concatenate([got[r]["logits"][pos] for r in range(size)])
        # the reduction tree differs (two partial sums instead of one sequential sum) and the fp16
        # key/value rounding can flip on it: binary32 tolerance, not bits
        assert np.linalg.norm(have - want) <= 1e-4 * np.linalg.norm(want)
        token = int(np.argmax(want))
        assert got[0]["tokens"][pos] == token and got[1]["tokens"][pos] == token


def test_exchange_sequence_keeps_alternating_slots_across_the_wrap():
    """The peer exchange picks one of two inbox slots by the parity of a 32-bit sequence number that
    lives on the device for the life of the model. Two exchanges in a row must never share a slot
    (a peer one exchange ahead would overwrite a packet not yet read), not even when the counter
    wraps, and 0 means "never written"."""
    from jitllm_b200 import _lib
    nxt = _lib.load().jl_debug_tp_next_sequence
    for seq in (1, 2, 3, 0x7FFFFFFF, 0x80000000, 0xFFFFFFFD, 0xFFFFFFFE, 0xFFFFFFFF):
        n = nxt(seq)
        assert n != 0
        assert (n & 1) != (seq & 1), hex(seq)
    assert nxt(0xFFFFFFFF) == 2 and nxt(5) == 6


def test_assembling_the_slices_gives_back_the_tensor():
    import jitllm_b200 as jl
    from jitllm_b200.tensor_parallel import assemble_tensor, shard_tensor
    cfg = jl.Configuration(dim=1024, hiddenDim=2048, numberOfLayers=1, numberOfHeads=8, numberOfKeyValueHeads=4,
                           vocabularySize=512, contextLength=16)
    for fmt in (jl.GGMLType.Q4_K, jl.GGMLType.Q8_0):
        for role in (jl.TensorRole.ATTENTION_QUERY, jl.TensorRole.ATTENTION_OUTPUT, jl.TensorRole.FFN_DOWN,
                     jl.TensorRole.OUTPUT, jl.TensorRole.TOKEN_EMBEDDING):
            rows, cols = cfg.matrix_shape(role)
            whole = jl.synth_tensor(fmt, rows * cols, seed=int(role) + 1)
            for size in (2, 4):
                shards = [shard_tensor(cfg, role, fmt, whole, jl.TensorParallel(r, size)) for r in range(size)]
                assert np.array_equal(assemble_tensor(cfg, role, shards), whole), (fmt, role, size)
