"""`query_runtime=` adapter for the reference's BaB driver.

`solve_bab_mlp(..., query_runtime=)` (boundflow/runtime/bab.py:631-639) hands every node
evaluation to `query_runtime.execute(module, requests)` and expects
`[(query_id, BoundQueryResult), ...]` in request order (bab.py:1005-1030, 1187-1250;
protocol: boundflow/runtime/bab_query_runtime.py:76-118, request / result types
boundflow/runtime/bab_query.py:192-279).  `CudaQueryRuntime.execute` does what the
reference's `execute_alpha_beta_query_batch` (boundflow/runtime/query_executor.py:96-197)
does -- stack the nodes' centres, split rows and warm starts, run the per-domain
alpha-beta loop once, slice the results per node -- on the CUDA backend, with one
difference: a node whose split assignment is empty gets `status="infeasible"` on its
own instead of failing the whole batch.  Chains on a box run on the fused whole-chain
loops; graphs that are not chains and L1 / L2 ball input sets go through
`run_alpha_beta_crown_mlp(per_batch_params=True)` on the same stacked batch.  The query's
`objective`, `spec_reduce`, `soft_tau`, `lb_weight` and `ub_weight` options reach the loop
(bab_query.py:860-864).

Requests are read by attribute only (`request.query.query_id`,
`request.query.bound_method`, `request.query.execution_options`, `request.payload.*`),
so the reference's own objects can be passed unchanged.  Results are the reference's
`BoundQueryResult` when that package is importable, else the mirror defined here.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Mapping, Optional, Sequence, Tuple

import torch

from .crown import (AlphaState, BetaState, alpha_crown_from_trace, branch_choices_from_trace, ibp_trace, needs_graph_path,
                    run_alpha_beta_crown_mlp)
from .ir import BoxPerturbation, InputSpec, input_mid_rad, lp_ball_of, normalize_input_spec


@dataclass(frozen=True)
class BoundQueryResult:
    """Mirror of boundflow/runtime/bab_query.py:231-262."""

    status: str
    lower: Optional[torch.Tensor]
    upper: Optional[torch.Tensor]
    branch: Optional[Tuple[str, int]]
    alpha_state_version: Optional[str]
    beta_state_version: Optional[str]
    alpha_by_relu_input: Mapping[str, torch.Tensor] = field(default_factory=dict)
    beta_by_relu_input: Mapping[str, torch.Tensor] = field(default_factory=dict)


def _result_type():
    try:  # the reference's own class when its package is present
        from boundflow.runtime.bab_query import BoundQueryResult as RefResult  # type: ignore

        return RefResult
    except Exception:
        return BoundQueryResult


def _rows_of_spec(spec: Any, rows: Sequence[int], ball) -> Any:
    """The input sets of the chosen nodes of a stacked spec."""
    idx = torch.as_tensor(list(rows), device=spec.center.device)
    if ball is not None:
        mk = InputSpec.l2 if int(ball[0]) == 2 else InputSpec.l1
        return mk(value_name=spec.value_name, center=spec.center[idx], eps=float(ball[1]))
    pert = spec.perturbation
    return InputSpec(spec.value_name, spec.center[idx], BoxPerturbation(lower=pert.lower[idx], upper=pert.upper[idx]))


def _method_name(query: Any) -> str:
    m = getattr(query, "bound_method", None)
    return str(getattr(m, "value", m))


def _option(options: Mapping[str, object], name: str, kind):
    if name not in options:
        raise ValueError(f"query execution option missing: {name}")
    return kind(options[name])


class CudaQueryRuntime:
    """Executes solver-provided query groups on the CUDA backend; owns no search control flow."""

    def __init__(self, *, max_batch_size: int = 8192):
        if max_batch_size <= 0:
            raise ValueError("max_batch_size must be positive")
        self.max_batch_size = int(max_batch_size)
        self._batches = 0
        self._queries = 0
        self._infeasible = 0

    # -- grouping -------------------------------------------------------------------------
    @staticmethod
    def _group_key(request: Any) -> tuple:
        q, p = request.query, request.payload
        spec = normalize_input_spec(p.input_spec)
        pert = spec.perturbation
        kind = "box" if hasattr(pert, "lower") else ("lp", str(getattr(pert, "p", None)), float(getattr(pert, "eps", 0.0)))
        c = p.linear_spec_c
        return (
            _method_name(q),
            tuple(sorted((k, repr(v)) for k, v in dict(q.execution_options).items())),
            kind,
            tuple(spec.center.shape[1:]),
            None if c is None else tuple(c.shape[-2:]),
            tuple(sorted(p.split_by_relu_input)),
        )

    def execute(self, module: Any, requests: Sequence[Any], *, now_us: Optional[int] = None) -> List[Tuple[str, Any]]:
        """One solver-selected group, results in the original order (bab_query_runtime.py:76-118)."""
        if not requests:
            return []
        groups: Dict[tuple, List[int]] = {}
        for i, r in enumerate(requests):
            groups.setdefault(self._group_key(r), []).append(i)
        out: List[Optional[Tuple[str, Any]]] = [None] * len(requests)
        for key, idx in groups.items():
            for s in range(0, len(idx), self.max_batch_size):
                part = idx[s : s + self.max_batch_size]
                results = self._execute_batch(module, [requests[i] for i in part], key[0])
                for i, res in zip(part, results):
                    out[i] = (requests[i].query.query_id, res)
        if any(o is None for o in out):
            raise ValueError("query runtime lost a query result")
        return [o for o in out if o is not None]

    # -- one homogeneous batch ------------------------------------------------------------
    def _execute_batch(self, module: Any, reqs: Sequence[Any], method: str) -> List[Any]:
        Result = _result_type()
        opts = dict(reqs[0].query.execution_options)
        steps = _option(opts, "alpha_steps", int)
        lr = _option(opts, "alpha_lr", float)
        alpha_init = _option(opts, "alpha_init", float)
        # objective / reduction options of the replay (bab_query.py:860-864, 882-886)
        kw = {"objective": str(opts.get("objective", "lower")), "spec_reduce": str(opts.get("spec_reduce", "mean")),
              "soft_tau": float(opts.get("soft_tau", 1.0)), "lb_weight": float(opts.get("lb_weight", 1.0)),
              "ub_weight": float(opts.get("ub_weight", 1.0))}
        D = len(reqs)
        first = normalize_input_spec(reqs[0].payload.input_spec)
        dev_in = first.center.device
        if needs_graph_path(module) or lp_ball_of(first) is not None:
            return self._execute_batch_general(module, reqs, method, opts, kw, steps, lr, alpha_init)
        # stacked input set: per-node boxes (or L-inf balls as boxes)
        los, ups = [], []
        for r in reqs:
            _m, _r, lo, up = input_mid_rad(r.payload.input_spec)
            if int(lo.shape[0]) != 1:
                raise ValueError("a BaB query bounds one node: its input set must have batch size 1")
            los.append(lo)
            ups.append(up)
        lo_b, up_b = torch.cat(los, dim=0), torch.cat(ups, dim=0)
        spec = InputSpec(first.value_name, (lo_b + up_b) / 2.0, BoxPerturbation(lower=lo_b, upper=up_b))
        # stacked specs
        cs = [r.payload.linear_spec_c for r in reqs]
        if all(c is None for c in cs):
            C = None
        elif any(c is None for c in cs):
            raise ValueError("query batch mixes implicit and explicit output specs")
        else:
            C = torch.cat([c.unsqueeze(0) if c.dim() == 2 else c for c in cs], dim=0)
        names = list(reqs[0].payload.split_by_relu_input)
        splits = {n: torch.stack([r.payload.split_by_relu_input[n].reshape(-1) for r in reqs], dim=0) for n in names}

        trace = ibp_trace(module, spec, relu_split_state=splits if splits else None)
        chain, device = trace.chain, trace.mid.device
        relu_names = chain.relu_input_names

        def stacked(source: str, default: float) -> List[torch.Tensor]:
            rows = []
            for name, n in zip(relu_names, chain.relu_widths):
                per = []
                for r in reqs:
                    warm = getattr(r.payload, source).get(name)
                    per.append(torch.full((n,), float(default), dtype=torch.float32, device=device) if warm is None
                               else warm.detach().to(device=device, dtype=torch.float32).reshape(n))
                rows.append(torch.stack(per, dim=0))
            return rows

        alpha0 = stacked("warm_alpha_by_relu_input", alpha_init)
        if C is None:
            n_out = 1
            for d in chain.output_shape:
                n_out *= int(d)
            C = torch.eye(n_out, dtype=torch.float32, device=device)
        best_b: Optional[List[torch.Tensor]] = None
        if method == "alpha-beta-CROWN":
            beta0 = stacked("warm_beta_by_relu_input", _option(opts, "beta_init", float))
            if splits:
                beta_splits = [splits.get(n) for n in relu_names]
                best_l, best_u, best_a, _last, _metric, best_b = alpha_crown_from_trace(
                    trace, C, alpha0, steps=steps, lr=lr, beta_splits=beta_splits, beta0=beta0, **kw)
            else:
                best_l, best_u, best_a, _last, _metric = alpha_crown_from_trace(trace, C, alpha0, steps=steps, lr=lr, **kw)
                best_b = beta0
            branches: List[Optional[Tuple[str, int]]] = branch_choices_from_trace(trace)
        elif method == "alpha-CROWN":
            # the reference replays these one node at a time with alpha shared across the node's single batch row
            # (bab_query.py:875-891); with one row per node that is the per-domain optimisation
            best_l, best_u, best_a, _last, _metric = alpha_crown_from_trace(trace, C, alpha0, steps=steps, lr=lr, **kw)
            branches = [None] * D
        else:
            raise ValueError(f"unsupported BaB query method: {method}")

        infeasible = trace.infeasible.to("cpu")  # one synchronisation per batch
        self._batches += 1
        self._queries += D
        results = []
        for i in range(D):
            if int(infeasible[i]) != 0:
                self._infeasible += 1
                # the alpha-beta path reports an empty node; the alpha-only replay rejects it (bab_query.py:894-909)
                status = "infeasible" if method == "alpha-beta-CROWN" else "rejected"
                results.append(Result(status=status, lower=None, upper=None, branch=None, alpha_state_version=None, beta_state_version=None))
                continue
            alpha_i = {n: a[i].reshape(tuple(s)).to(dev_in).clone() for n, a, s in zip(relu_names, best_a, chain.relu_shapes)}
            beta_i = {} if best_b is None else {n: b[i].reshape(tuple(s)).to(dev_in).clone() for n, b, s in zip(relu_names, best_b, chain.relu_shapes)}
            results.append(Result(
                status="ok", lower=best_l[i : i + 1].to(dev_in).clone(), upper=best_u[i : i + 1].to(dev_in).clone(), branch=branches[i],
                alpha_state_version=None, beta_state_version=None, alpha_by_relu_input=alpha_i, beta_by_relu_input=beta_i))
        return results

    # -- graphs that are not chains, and L1 / L2 ball inputs: the whole-query functions --------------
    def _execute_batch_general(self, module: Any, reqs: Sequence[Any], method: str, opts: Mapping[str, object], kw: Mapping[str, object],
                               steps: int, lr: float, alpha_init: float) -> List[Any]:
        """The same stacking through `run_alpha_beta_crown_mlp(per_batch_params=True)`, which walks non-chain graphs and
        takes Lp balls.  A batch with an empty node raises there; its nodes are then evaluated one by one so that only the
        empty ones are reported."""
        Result = _result_type()
        D = len(reqs)
        first = normalize_input_spec(reqs[0].payload.input_spec)
        dev_in = first.center.device
        ball = lp_ball_of(first)
        specs = [normalize_input_spec(r.payload.input_spec) for r in reqs]
        if any(int(sp.center.shape[0]) != 1 for sp in specs):
            raise ValueError("a BaB query bounds one node: its input set must have batch size 1")
        if ball is not None:
            mk = InputSpec.l2 if int(ball[0]) == 2 else InputSpec.l1
            spec = mk(value_name=first.value_name, center=torch.cat([sp.center for sp in specs], dim=0), eps=float(ball[1]))
        else:
            boxes = [input_mid_rad(sp) for sp in specs]
            lo_b, up_b = torch.cat([b[2] for b in boxes], dim=0), torch.cat([b[3] for b in boxes], dim=0)
            spec = InputSpec(first.value_name, (lo_b + up_b) / 2.0, BoxPerturbation(lower=lo_b, upper=up_b))
        cs = [r.payload.linear_spec_c for r in reqs]
        if all(c is None for c in cs):
            C = None
        elif any(c is None for c in cs):
            raise ValueError("query batch mixes implicit and explicit output specs")
        else:
            C = torch.cat([c.unsqueeze(0) if c.dim() == 2 else c for c in cs], dim=0)
        names = list(reqs[0].payload.split_by_relu_input)
        splits = {n: torch.stack([r.payload.split_by_relu_input[n].reshape(-1) for r in reqs], dim=0) for n in names}

        def warm(source: str, default: float):
            """Stacked warm starts; a node without one takes the default value, a ReLU no node warms keeps the loop's own start."""
            seen: Dict[str, torch.Tensor] = {}
            for r in reqs:
                for n, t in getattr(r.payload, source).items():
                    if t is not None:
                        seen.setdefault(n, t)
            out = {}
            for n, like in seen.items():
                rows = []
                for r in reqs:
                    t = getattr(r.payload, source).get(n)
                    rows.append(torch.full((like.numel(),), float(default), dtype=torch.float32, device=like.device) if t is None
                                else t.detach().to(dtype=torch.float32).reshape(-1))
                out[n] = torch.stack(rows, dim=0)
            return out

        with_beta = method == "alpha-beta-CROWN"
        if method not in ("alpha-beta-CROWN", "alpha-CROWN"):
            raise ValueError(f"unsupported BaB query method: {method}")
        beta_init = _option(opts, "beta_init", float) if with_beta else 0.0
        wa, wb = warm("warm_alpha_by_relu_input", alpha_init), (warm("warm_beta_by_relu_input", beta_init) if with_beta else {})

        def run(rows: Sequence[int]):
            sub = spec if len(rows) == D else _rows_of_spec(spec, rows, ball)
            idx = torch.as_tensor(list(rows))
            return run_alpha_beta_crown_mlp(
                module, sub, linear_spec_C=None if C is None else C[idx.to(C.device)],
                relu_split_state={n: v[idx.to(v.device)] for n, v in splits.items()} if splits else None, steps=steps, lr=lr, alpha_init=alpha_init,
                beta_init=beta_init, warm_start_alpha=AlphaState({n: v[idx.to(v.device)] for n, v in wa.items()}) if wa else None,
                warm_start_beta=BetaState({n: v[idx.to(v.device)] for n, v in wb.items()}) if wb else None, per_batch_params=True,
                optimize_beta=bool(with_beta and splits), **kw)

        self._batches += 1
        self._queries += D
        empty = Result(status="infeasible" if with_beta else "rejected", lower=None, upper=None, branch=None, alpha_state_version=None,
                       beta_state_version=None)
        try:
            parts = [(list(range(D)), run(list(range(D))))]
        except ValueError:
            parts = []
            for i in range(D):
                try:
                    parts.append(([i], run([i])))
                except ValueError:
                    parts.append(([i], None))
        results: List[Any] = [None] * D
        for rows, res in parts:
            if res is None:
                self._infeasible += len(rows)
                for i in rows:
                    results[i] = empty
                continue
            bounds, a_state, b_state, stats = res
            if getattr(stats, "feasibility", "unknown") == "infeasible":   # the single-node certificate fired
                self._infeasible += len(rows)
                for i in rows:
                    results[i] = empty
                continue
            choices = getattr(stats, "branch_choices", None)
            for k, i in enumerate(rows):
                alpha_i = {n: v[k].to(dev_in).clone() for n, v in a_state.alpha_by_relu_input.items()}
                beta_i = {n: v[k].to(dev_in).clone() for n, v in b_state.beta_by_relu_input.items()} if with_beta else {}
                results[i] = Result(status="ok", lower=bounds.lower[k : k + 1].to(dev_in).clone(), upper=bounds.upper[k : k + 1].to(dev_in).clone(),
                                    branch=(choices[k] if (with_beta and choices) else None), alpha_state_version=None, beta_state_version=None,
                                    alpha_by_relu_input=alpha_i, beta_by_relu_input=beta_i)
        return results

    def audit(self) -> Dict[str, object]:
        """Accounting in the spirit of SameSolverQueryRuntime.audit (bab_query_runtime.py:120-139)."""
        return {"batches": self._batches, "queries": self._queries, "infeasible_queries": self._infeasible,
                "backend": "b200_cuda", "max_batch_size": self.max_batch_size}
