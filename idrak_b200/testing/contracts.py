"""Contract suites: what any implementation of a pluggable piece must do, stated as runnable checks.

A suite has fixed cases (the corner cases someone once got wrong), seeded random cases, and ``run(implementation)``
which returns the list of violated clauses (empty = conforms). Every suite names a reference implementation and a
deliberately broken twin: the suite's own test is that the reference passes and the twin is rejected, so a suite that
checks nothing cannot ship.

Reference: ContractSuite<T> (src/Idrak.Abstraction.Testing/ContractSuite.cs:38) and the suites under
src/Idrak.Abstraction.Testing/Contracts (sampler, tokenizer, RoPE scaling, codecs, collectives, transport).
"""
from __future__ import annotations

import math
from typing import Any, Callable, Dict, List, Sequence

import torch


class ContractSuite:
    """Base: subclasses give ``fixed_cases``, ``random_case`` and ``verify``."""
    name = "contract"

    def fixed_cases(self) -> List[Any]:
        return []

    def random_case(self, seed: int) -> Any:
        raise NotImplementedError

    def verify(self, implementation, case) -> List[str]:
        raise NotImplementedError

    def reference(self):
        raise NotImplementedError

    def broken(self):
        raise NotImplementedError

    def run(self, implementation, random_cases: int = 16, seed: int = 0) -> List[str]:
        problems: List[str] = []
        cases = list(self.fixed_cases()) + [self.random_case(seed + i) for i in range(random_cases)]
        for i, case in enumerate(cases):
            try:
                problems += [f"{self.name} case {i}: {p}" for p in self.verify(implementation, case)]
            except Exception as e:      # an implementation that throws on a legal case violates the contract
                problems.append(f"{self.name} case {i}: raised {type(e).__name__}: {e}")
        return problems

    def self_test(self) -> List[str]:
        """The suite's own check: the reference conforms, the broken twin does not."""
        out = [f"reference rejected: {p}" for p in self.run(self.reference())]
        if not self.run(self.broken()):
            out.append(f"{self.name}: the broken twin passed - the suite checks too little")
        return out


# --------------------------------------------------------------------------- sampler
class SamplerContract(ContractSuite):
    """``sample(logits [rows, V], temperature, top_k, top_p, min_p, uniforms) -> ids [rows]``.

    Clauses: ids inside the vocabulary; top_k = 1 gives the arg-max with ties to the lowest id; the pick lies inside the
    top-k set; with top_p -> 0 or min_p = 1 only the arg-max survives; the same uniforms give the same ids."""
    name = "sampler"

    def fixed_cases(self):
        tie = torch.zeros(2, 40)
        tie[0, [5, 9, 30]] = 3.0          # three-way tie: lowest id wins
        tie[1, 39] = 1.0
        return [dict(logits=tie, top_k=1, top_p=1.0, min_p=0.0, temperature=1.0, u=0.5),
                dict(logits=torch.full((1, 16), -1e4), top_k=4, top_p=0.9, min_p=0.0, temperature=0.7, u=0.99)]

    def random_case(self, seed):
        g = torch.Generator().manual_seed(seed)
        rows, V = int(torch.randint(1, 6, (1,), generator=g)), int(torch.randint(8, 300, (1,), generator=g))
        return dict(logits=torch.randn(rows, V, generator=g) * 3, top_k=int(torch.randint(1, 20, (1,), generator=g)),
                    top_p=float(torch.rand(1, generator=g)) * 0.9 + 0.1, min_p=float(torch.rand(1, generator=g)) * 0.2,
                    temperature=float(torch.rand(1, generator=g)) + 0.3, u=float(torch.rand(1, generator=g)))

    def verify(self, sample, c):
        logits = c["logits"]
        rows, V = logits.shape

        def call(top_k, top_p, min_p, u):
            return sample(logits, torch.full((rows,), c["temperature"]), torch.full((rows,), top_k, dtype=torch.int32),
                          torch.full((rows,), top_p), torch.full((rows,), min_p), torch.full((rows,), u)).long()
        out: List[str] = []
        ids = call(c["top_k"], c["top_p"], c["min_p"], c["u"])
        if ids.shape != (rows,) or int(ids.min()) < 0 or int(ids.max()) >= V:
            return ["ids outside the vocabulary"]
        if not torch.equal(ids, call(c["top_k"], c["top_p"], c["min_p"], c["u"])):
            out.append("same uniforms, different ids")
        order = torch.sort(logits, dim=-1, descending=True, stable=True).indices
        for r in range(rows):
            if int(ids[r]) not in order[r, : c["top_k"]].tolist():
                out.append("pick outside the top-k set")
                break
        first = order[:, 0]
        for what, got in (("top_k = 1", call(1, 1.0, 0.0, c["u"])), ("top_p -> 0", call(c["top_k"], 1e-6, 0.0, c["u"])),
                          ("min_p = 1", call(c["top_k"], 1.0, 1.0, 0.0))):
            if not torch.equal(got, first):
                out.append(f"{what} must give the arg-max (ties: lowest id)")
        return out

    def reference(self):
        from ..ops.decode import sample_rows_reference
        return lambda logits, t, k, p, m, u: sample_rows_reference(logits, logits.shape[1], t, k, p, m, u)

    def broken(self):
        ref = self.reference()

        def twin(logits, t, k, p, m, u):       # ties go to the highest id
            return ref(logits.flip(-1), t, k, p, m, u).mul(-1).add(logits.shape[1] - 1)
        return twin


# --------------------------------------------------------------------------- tokenizer
class TokenizerContract(ContractSuite):
    """``encode(text) -> ids``, ``decode(ids) -> text``: round trip, determinism, concatenation of decodes."""
    name = "tokenizer"
    _TEXTS = ["", " ", "hello world", "  leading and trailing  ", "naïve café — ünïcödé", "a\nb\r\n\tc",
              "1234567890" * 5, "日本語のテキスト", "emoji 🙂🙃", "x" * 300]

    def fixed_cases(self):
        return list(self._TEXTS)

    def random_case(self, seed):
        g = torch.Generator().manual_seed(seed)
        alphabet = "abcdefghij klmnop\nqrstuvwxyzABC.,;!?0123456789éü😀"
        n = int(torch.randint(1, 80, (1,), generator=g))
        return "".join(alphabet[int(i)] for i in torch.randint(0, len(alphabet), (n,), generator=g))

    def verify(self, tok, text):
        out = []
        ids = list(tok.encode(text))
        if ids != list(tok.encode(text)):
            out.append("encode is not deterministic")
        if tok.decode(ids) != text:
            out.append(f"decode(encode(x)) != x for {text[:30]!r}")
        if any((not isinstance(i, int)) or i < 0 or i >= tok.vocab_size for i in ids):
            out.append("id outside the vocabulary")
        return out

    def reference(self):
        return _ByteTokenizer()

    def broken(self):
        return _ByteTokenizer(drop_spaces=True)


class _ByteTokenizer:
    vocab_size = 256

    def __init__(self, drop_spaces=False):
        self.drop = drop_spaces

    def encode(self, text):
        return [b for b in text.encode("utf-8") if not (self.drop and b == 32)]

    def decode(self, ids):
        return bytes(ids).decode("utf-8", errors="replace")


# --------------------------------------------------------------------------- rope scaling
class RopeScalingContract(ContractSuite):
    """``inv_freq(spec, head_dim, seq_len) -> (frequencies, attention factor)``: one positive frequency per pair,
    non-increasing; a factor of 1 (or no scaling) leaves theta^(-2k/d); no frequency grows under scaling."""
    name = "rope-scaling"

    def fixed_cases(self):
        return [dict(scaling=None, factor=1.0, D=64, S=128), dict(scaling="linear", factor=4.0, D=128, S=4096),
                dict(scaling="llama3", factor=8.0, D=128, S=16384), dict(scaling="yarn", factor=4.0, D=64, S=16384),
                dict(scaling="dynamic", factor=2.0, D=64, S=20000)]

    def random_case(self, seed):
        g = torch.Generator().manual_seed(seed)
        kinds = [None, "linear", "llama3", "yarn", "dynamic"]
        return dict(scaling=kinds[int(torch.randint(0, 5, (1,), generator=g))],
                    factor=float(torch.rand(1, generator=g)) * 7 + 1, D=[64, 128][int(torch.randint(0, 2, (1,), generator=g))],
                    S=int(torch.randint(16, 40000, (1,), generator=g)))

    def verify(self, inv_freq, c):
        from ..models.spec import RopeSettings
        spec = RopeSettings(theta=10000.0, scaling=c["scaling"], factor=c["factor"], original_max_positions=8192)
        inv, mscale = inv_freq(spec, c["D"], c["S"])
        plain = [10000.0 ** (-2.0 * k / c["D"]) for k in range(c["D"] // 2)]
        out = []
        if len(inv) != c["D"] // 2 or any(not (f > 0 and math.isfinite(f)) for f in inv):
            return ["needs one positive finite frequency per pair"]
        if any(inv[i + 1] > inv[i] * (1 + 1e-9) for i in range(len(inv) - 1)):
            out.append("frequencies must not increase along the pairs")
        if any(f > p * (1 + 1e-6) for f, p in zip(inv, plain)):
            out.append("scaling must not raise a frequency")
        if c["scaling"] is None and any(abs(f - p) > 1e-12 * max(p, 1e-30) + 1e-15 for f, p in zip(inv, plain)):
            out.append("no scaling must leave theta^(-2k/d)")
        if not (mscale > 0):
            out.append("attention factor must be positive")
        return out

    def reference(self):
        return lambda spec, D, S: spec.inv_freq(D, S)

    def broken(self):
        def twin(spec, D, S):
            inv, m = spec.inv_freq(D, S)
            return [f * (spec.factor if spec.scaling == "linear" else 1.0) ** 2 for f in inv], m   # multiplies instead
        return twin


# --------------------------------------------------------------------------- collectives
class CollectiveContract(ContractSuite):
    """``all_reduce(list of per-rank tensors) -> list of per-rank results``: every rank ends with the same bits and that
    value is the sum; ``reduce_scatter`` pieces concatenate to that sum; ``all_gather`` concatenates in rank order."""
    name = "collectives"

    def fixed_cases(self):
        return [dict(world=1, n=5, seed=1), dict(world=2, n=1, seed=2), dict(world=3, n=10, seed=3),
                dict(world=4, n=1025, seed=4), dict(world=5, n=3, seed=5)]      # fewer elements than ranks included

    def random_case(self, seed):
        g = torch.Generator().manual_seed(seed)
        return dict(world=int(torch.randint(1, 9, (1,), generator=g)), n=int(torch.randint(1, 3000, (1,), generator=g)),
                    seed=seed)

    def verify(self, impl, c):
        g = torch.Generator().manual_seed(c["seed"])
        parts = [torch.randn(c["n"], generator=g) for _ in range(c["world"])]
        want = torch.stack(parts).double().sum(0)
        out = []
        got = impl["all_reduce"]([p.clone() for p in parts])
        if any(not torch.equal(got[0], t) for t in got[1:]):
            out.append("all_reduce: ranks end with different bits")
        if (got[0].double() - want).abs().max() > 1e-5 * max(1.0, float(want.abs().max())):
            out.append("all_reduce: not the sum")
        if "reduce_scatter" in impl:
            pieces = impl["reduce_scatter"]([p.clone() for p in parts])
            cat = torch.cat(list(pieces))
            if cat.shape != want.shape or (cat.double() - want).abs().max() > 1e-5 * max(1.0, float(want.abs().max())):
                out.append("reduce_scatter: pieces do not concatenate to the sum")
        if "all_gather" in impl:
            full = impl["all_gather"]([p.clone() for p in parts])
            if any(not torch.equal(f, torch.cat(parts)) for f in full):
                out.append("all_gather: not the rank-order concatenation on every rank")
        return out

    @staticmethod
    def _over_simulator(kind: str, corrupt: bool = False) -> Dict[str, Callable]:
        """The host collectives of the package run over in-process threads, one per rank."""
        from ..parallel.host_collectives import create
        from ..parallel.transport import MemoryTransport

        def run(method):
            def go(parts):
                world = len(parts)
                hub = MemoryTransport.hub(world, corrupt=corrupt)
                return hub.run(lambda rank, tr: getattr(create(kind, tr.as_exchange()), method)(parts[rank]))
            return go
        return {"all_reduce": run("all_reduce"), "reduce_scatter": run("reduce_scatter"), "all_gather": run("all_gather")}

    def reference(self):
        return self._over_simulator("ring")

    def broken(self):
        return self._over_simulator("ring", corrupt=True)


# --------------------------------------------------------------------------- gradient codecs
class CodecContract(ContractSuite):
    """``encode(x) -> payload``, ``decode(payload) -> y``: y has x's shape; |y - x| within the codec's stated bound of
    max|x|; zeros stay zeros; with error feedback the running sum of what was sent tracks the running sum of x."""
    name = "codec"

    def fixed_cases(self):
        return [torch.zeros(17), torch.ones(1), torch.tensor([1e-8, -1e4, 3.0, 0.0]), torch.linspace(-2, 2, 1000)]

    def random_case(self, seed):
        g = torch.Generator().manual_seed(seed)
        return torch.randn(int(torch.randint(1, 5000, (1,), generator=g)), generator=g) * float(torch.rand(1, generator=g) * 10)

    def verify(self, codec, x):
        y = codec["decode"](codec["encode"](x))
        out = []
        if y.shape != x.shape:
            return ["shape changed"]
        peak = float(x.abs().max())
        if float((y - x).abs().max()) > codec["bound"] * peak + 1e-30:
            out.append(f"error above {codec['bound']} of the largest magnitude")
        if peak == 0 and float(y.abs().max()) != 0:
            out.append("zeros must stay zeros")
        carry, sent, total = torch.zeros_like(x), torch.zeros_like(x), torch.zeros_like(x)
        for _ in range(8):
            want = x + carry
            y = codec["decode"](codec["encode"](want))
            carry = want - y
            sent += y
            total += x
        if float((sent + carry - total).abs().max()) > 1e-4 * max(1.0, peak * 8):
            out.append("error feedback does not conserve the sum")
        return out

    def reference(self):
        def enc(x):
            s = float(x.abs().max()) / 127 or 1.0
            return (torch.clamp(torch.round(x / s), -127, 127).to(torch.int8), s)
        return {"encode": enc, "decode": lambda p: p[0].float() * p[1], "bound": 0.5 / 127 + 1e-6}

    def broken(self):
        ref = self.reference()
        return {"encode": lambda x: ref["encode"](x.abs()), "decode": ref["decode"], "bound": ref["bound"]}   # loses the sign



# --------------------------------------------------------------------------- transport
def run_ranks(world: int, make_transport: Callable[[int], Any], fn: Callable[[int, Any], Any], timeout: float = 60.0):
    """One thread per rank: builds the rank's transport, runs ``fn(rank, transport)``, closes it (orderly only when
    ``fn`` returned). Returns (results, errors) in rank order."""
    import threading
    results, errors = [None] * world, [None] * world

    def main(r):
        t = None
        try:
            t = make_transport(r)
            results[r] = fn(r, t)
            t.close(True)
        except BaseException as e:
            errors[r] = e
            if t is not None:
                t.close(False)
    threads = [threading.Thread(target=main, args=(r,), daemon=True) for r in range(world)]
    for t in threads:
        t.start()
    for t in threads:
        t.join(timeout)
    return results, errors


class TransportContract(ContractSuite):
    """``factory(world) -> make_transport(rank)``. Clauses: messages between a pair arrive in order, with their dtype
    and values intact, empty and large ones included; a barrier lets nobody through early; a rank that leaves makes
    its peers' ``recv`` raise ``PeerLost`` naming it, ``orderly`` telling an announced leave from a drop."""
    name = "transport"

    def fixed_cases(self):
        return [dict(world=2, sizes=[0, 1, 70000], seed=1, leave=None), dict(world=3, sizes=[5, 5], seed=2, leave=None),
                dict(world=3, sizes=[3], seed=3, leave=("bye", 1)), dict(world=2, sizes=[3], seed=4, leave=("drop", 0))]

    def random_case(self, seed):
        g = torch.Generator().manual_seed(seed)
        return dict(world=int(torch.randint(2, 5, (1,), generator=g)),
                    sizes=[int(x) for x in torch.randint(0, 5000, (int(torch.randint(1, 5, (1,), generator=g)),), generator=g)],
                    seed=seed, leave=None)

    def verify(self, factory, c):
        from ..parallel.transport import PeerLost
        world, sizes = c["world"], c["sizes"]
        dtypes = [torch.float32, torch.bfloat16, torch.int32, torch.int64]

        def message(src, dst, i):
            g = torch.Generator().manual_seed(c["seed"] * 1000 + src * 100 + dst * 10 + i)
            return (torch.randn(sizes[i], generator=g) * 100).to(dtypes[(src + i) % 4])

        leave = c["leave"]

        def body(rank, t):
            bad = []
            if leave is not None and rank == leave[1]:
                if leave[0] == "drop":
                    raise RuntimeError("rank stops without a word")
                return bad                                            # orderly: returns at once, close(True) follows
            def send_all():          # on its own thread: a transport with bounded buffering may make a sender wait
                try:
                    for i in range(len(sizes)):
                        for d in range(world):
                            if d != rank and not (leave and d == leave[1]):
                                t.send(d, message(rank, d, i))
                except BaseException as e:
                    bad.append(f"send raised {type(e).__name__}: {e}")
            import threading
            sender = threading.Thread(target=send_all, daemon=True)
            sender.start()
            for s in range(world):
                if s == rank:
                    continue
                if leave and s == leave[1]:
                    try:
                        t.recv(s, 10.0)
                        bad.append("recv from a rank that left returned a message")
                    except PeerLost as e:
                        if e.rank != s:
                            bad.append(f"PeerLost names rank {e.rank}, the one that left is {s}")
                        if e.orderly != (leave[0] == "bye"):
                            bad.append("orderly flag does not tell an announced leave from a drop")
                    continue
                for i in range(len(sizes)):
                    got, want = t.recv(s, 20.0), message(s, rank, i)
                    if got.dtype != want.dtype or got.shape != want.shape or not torch.equal(got, want):
                        bad.append(f"message {i} from rank {s} arrived changed or out of order")
            sender.join(30.0)
            if leave is None:
                t.barrier(20.0)
            return bad

        results, errors = run_ranks(world, factory(world), body)
        out = []
        for r in range(world):
            if errors[r] is not None and not (leave and r == leave[1] and leave[0] == "drop"):
                out.append(f"rank {r} raised {type(errors[r]).__name__}: {errors[r]}")
            out += results[r] or []
        return out

    def reference(self):
        from ..parallel.transport import MemoryTransport

        def factory(world):
            hub = MemoryTransport.hub(world)
            return lambda r: hub.ends[r]
        return factory

    def broken(self):
        from ..parallel.transport import MemoryTransport

        def factory(world):
            hub = MemoryTransport.hub(world, corrupt=True)
            return lambda r: hub.ends[r]
        return factory


SUITES: Dict[str, Callable[[], ContractSuite]] = {
    "sampler": SamplerContract, "tokenizer": TokenizerContract, "rope-scaling": RopeScalingContract,
    "collectives": CollectiveContract, "codec": CodecContract, "transport": TransportContract,
}
