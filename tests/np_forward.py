"""A second, independent statement of the Llama CPU forward pass in numpy binary32, written from
the reference's own inlined copy in
src/test/java/org/beehive/jitllm/inference/op/LlamaCpuOperationEquivalenceTest.java:201-338
(F32 weights, fp16 key/value cache, sequential sums). np.cumsum over float32 accumulates strictly
left to right, which is the order of FloatTensor.scalarDot / reduce."""
import numpy as np

F = np.float32


def seq_sum(v: np.ndarray) -> np.float32:
    return np.cumsum(v.astype(F), dtype=F)[-1] if v.size else F(0)


def rmsnorm(x, w, eps):
    ss = seq_sum((x * x).astype(F))
    ss = F(ss / F(x.size))
    ss = F(ss + F(eps))
    ss = F(1.0 / np.sqrt(np.float64(ss)))
    return (w * (ss * x).astype(F)).astype(F)


def matvec(w, x, rows, cols):
    prod = (w.reshape(rows, cols) * x[None, :]).astype(F)
    return np.cumsum(prod, axis=1, dtype=F)[:, -1]


class NpLlama:
    def __init__(self, cfg, w):
        self.c, self.w = cfg, w
        self.kc = np.zeros((cfg["layers"], cfg["ctx"], cfg["kv_dim"]), dtype=np.float16)
        self.vc = np.zeros_like(self.kc)

    def forward(self, token, pos):
        c, w = self.c, self.w
        dim, hs, kv_dim, heads = c["dim"], c["head"], c["kv_dim"], c["heads"]
        kv_mul = heads // c["kv_heads"]
        x = w["emb"][token * dim:(token + 1) * dim].copy()
        for l in range(c["layers"]):
            xb = rmsnorm(x, w["att_norm"][l], c["eps"])
            q = matvec(w["wq"][l], xb, dim, dim)
            k = matvec(w["wk"][l], xb, kv_dim, dim)
            v = matvec(w["wv"][l], xb, kv_dim, dim)
            for i in range(0, dim, 2):
                fcr = w["cr"][pos * (hs // 2) + (i % hs) // 2]
                fci = w["ci"][pos * (hs // 2) + (i % hs) // 2]
                for vec in ((q, k) if i < kv_dim else (q,)):
                    v0, v1 = vec[i], vec[i + 1]
                    vec[i] = F(F(v0 * fcr) - F(v1 * fci))
                    vec[i + 1] = F(F(v0 * fci) + F(v1 * fcr))
            self.kc[l, pos] = k.astype(np.float16)
            self.vc[l, pos] = v.astype(np.float16)
            out = np.zeros(dim, dtype=F)
            for h in range(heads):
                kh = self.kc[l, :pos + 1, (h // kv_mul) * hs:(h // kv_mul + 1) * hs].astype(F)
                vh = self.vc[l, :pos + 1, (h // kv_mul) * hs:(h // kv_mul + 1) * hs].astype(F)
                qh = q[h * hs:(h + 1) * hs]
                sc = np.cumsum((qh[None, :] * kh).astype(F), axis=1, dtype=F)[:, -1]
                sc = (sc / F(np.sqrt(np.float64(hs)))).astype(F)
                mx = sc.max()
                e = np.exp((sc - mx).astype(F).astype(np.float64)).astype(F)
                a = (e / seq_sum(e)).astype(F)
                acc = np.zeros(hs, dtype=F)
                for t in range(pos + 1):
                    acc = ((a[t] * vh[t]).astype(F) + acc).astype(F)
                out[h * hs:(h + 1) * hs] = acc
            x = (x + matvec(w["wo"][l], out, dim, dim)).astype(F)
            xb = rmsnorm(x, w["ffn_norm"][l], c["eps"])
            g = matvec(w["w1"][l], xb, c["hidden"], dim)
            u = matvec(w["w3"][l], xb, c["hidden"], dim)
            g = (g / (1.0 + np.exp(-g.astype(np.float64))).astype(F)).astype(F)
            hb = (g * u).astype(F)
            x = (x + matvec(w["w2"][l], hb, dim, c["hidden"])).astype(F)
        x = rmsnorm(x, w["final_norm"], c["eps"])
        return matvec(w["wcls"], x, c["vocab"], dim)
