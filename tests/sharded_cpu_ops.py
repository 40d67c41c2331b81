"""float64 CPU implementation of the shard-local steps (test infrastructure): the same formulas as
oracle/tier2_torch.py, cut where the sharded stack puts its collectives."""
import numpy as np
import torch

from oracle import tier2_torch as t2

T = t2.T


class CpuShardOps:
    def __init__(self, rows, length, ranks, eps=1e-5):
        self.R, self.N, self.G, self.eps = rows, length, ranks, eps
        self._zn = None

    def new_product(self):
        return torch.zeros((self.R, self.N, 0), dtype=torch.float64)   # sized on first chunk

    def triangle_project(self, z, mask, w):
        zn = t2.ln(z, w["layerNormInWeight"], w["layerNormInBias"], self.eps)
        lin = lambda x, k: x @ T(w[f"linear{k}Weight"]).T + T(w[f"linear{k}Bias"])
        m = mask[..., None]
        a = lin(zn, "AP") * torch.sigmoid(lin(zn, "AG")) * m
        b = lin(zn, "BP") * torch.sigmoid(lin(zn, "BG")) * m
        self._x = torch.zeros((self.R, self.N, a.shape[-1]), dtype=torch.float64)
        return a, b

    def triangle_contract(self, a, b_chunk, x, chunk, w):
        self._x[:, chunk * self.R:(chunk + 1) * self.R, :] = torch.einsum("ikc,jkc->ijc", a, b_chunk)

    def triangle_output(self, x, z, w):
        lin = lambda v, k: v @ T(w[f"linear{k}Weight"]).T + T(w[f"linear{k}Bias"])
        zn = t2.ln(z, w["layerNormInWeight"], w["layerNormInBias"], self.eps)
        xn = t2.ln(self._x, w["layerNormOutWeight"], w["layerNormOutBias"], self.eps)
        z += lin(xn, "Z") * torch.sigmoid(lin(zn, "G"))

    def attention_project(self, z, t):
        w = t["attention"]
        n = t2.ln(z, w["queryNormScale"], w["queryNormOffset"], self.eps)
        q, k, v = n @ T(w["queryWeight"]), n @ T(w["keyWeight"]), n @ T(w["valueWeight"])
        g = torch.sigmoid(n @ T(w["gatingWeight"]) + T(w["gatingBias"]))
        bias = (n @ T(t["pairBias"]["projectionWeight"])).permute(2, 0, 1).contiguous()     # [H][local q][k]
        return q, k, v, g, bias

    def attention_core(self, q, k, v, g, bias_all, mask, t):
        heads = t["heads"]
        bias = bias_all.permute(1, 0, 2, 3).reshape(heads, self.N, self.N)                  # [H][q][k], ranks in row order
        extra = (1e9 * (mask - 1.0))[:, None, None, :] + bias[None]
        logits, vh = t2._attend(q, k, v, extra, heads)
        logits = logits.clamp(-1e8, 1e8)
        p = torch.softmax(logits.to(torch.float32).to(torch.float64), -1)
        return (p @ vh).permute(0, 2, 1, 3).reshape(self.R, self.N, -1) * g

    # -- channel-sharded triangle multiplication and scattered bias, exchanged through `comm`
    #    (what the GPU path does with stores into the peers' memory)

    def exchange_triangle_project(self, z, mask, w, ex, comm):
        a, b = self.triangle_project(z, mask, w)                   # [R][N][c]
        G, c = comm.world, a.shape[-1]
        cpr = c // G

        def to_channel_owner(t):       # rank g receives channels [g cpr, (g+1) cpr) of every rank's rows
            send = t.reshape(self.R, self.N, G, cpr).permute(2, 0, 1, 3).contiguous()      # [dest][r][k][cpr]
            recv = comm.all_to_all(send)                                                   # [src][r][k][cpr]
            return recv.reshape(G * self.R, self.N, cpr)                                   # [n][k][cpr]: all rows

        self._a_cs, self._b_cs = to_channel_owner(a), to_channel_owner(b)

    def exchange_triangle_contract(self, w, ex, comm, incoming):
        a, b = self._a_cs, self._b_cs
        x = torch.einsum("kjc,kic->ijc", a, b) if incoming else torch.einsum("ikc,jkc->ijc", a, b)   # [N][N][cpr]
        G = comm.world
        send = x.reshape(G, self.R, self.N, -1).contiguous()                                # [dest][r][j][cpr]
        recv = comm.all_to_all(send)                                                        # [src = channel block][r][j][cpr]
        self._x = recv.permute(1, 2, 0, 3).reshape(self.R, self.N, -1)                      # channels back in order
        return self._x

    def exchange_attention_project(self, z, t, ex, comm):
        q, k, v, g, bias = self.attention_project(z, t)
        return q, k, v, g, comm.all_gather(bias)

    def attention_output(self, o, z, t):
        w = t["attention"]
        z += o @ T(w["outputWeight"]) + T(w["outputBias"])

    def transition(self, z, w):
        z += torch.from_numpy(t2.transition_af2(z.numpy(), w, self.eps))


def block_weights(w):
    return {"triangle_outgoing": w["triangleMultiplicationOutgoing"], "triangle_incoming": w["triangleMultiplicationIncoming"],
            "attention_starting": w["triangleAttentionStarting"], "attention_ending": w["triangleAttentionEnding"],
            "transition": w["pairTransition"]}
