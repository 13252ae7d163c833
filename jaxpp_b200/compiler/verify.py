"""Static checks on a compiled program (the reference only has ``check_jaxpr`` behind
``JAXPP_ENABLE_CHECK_JAXPR``, src/jaxpp/jaxpr_utils.py:32-35, and ``check_scalar_jaxprs``,
src/jaxpp/core.py:3524).

* every value is defined on a rank before that rank uses it and is not used after its delete;
* the per-rank programs cannot deadlock: they are replayed with *blocking rendezvous* point-to-point
  semantics (a send completes only when the matching receive has been reached, per channel in
  order — the strictest behaviour NCCL p2p may show) and blocking collectives;
* every transfer id is sent once and received once, collectives are joined by all their ranks.
"""
from __future__ import annotations

from collections import defaultdict

from .program import (Accum, AllGather, AllReduce, Delete, LoopIndex, Program, RunTask, Slice, Transfer)


class ProgramError(AssertionError):
    pass


def _uses_defs(ins, rank):
    if isinstance(ins, RunTask):
        return list(ins.ins), [v for v in ins.outs if v >= 0] + [h[2] for h in ins.hooks]
    if isinstance(ins, Slice):
        return [ins.src], [ins.out]
    if isinstance(ins, LoopIndex):
        return [], [ins.out]
    if isinstance(ins, Accum):
        return [ins.val], [ins.acc]
    if isinstance(ins, Transfer):
        return (list(ins.vids), []) if ins.rank == rank else ([], list(ins.vids))
    if isinstance(ins, AllReduce):
        return list(ins.local), [ins.out]
    if isinstance(ins, AllGather):
        return list(ins.local.values()), [ins.out]
    return [], []


def verify_program(prog: Program) -> dict:
    # ---- def-before-use / use-after-delete per rank ------------------------------------------------
    for rank in range(prog.n_ranks):
        live = {vid for vid, ranks in prog.inputs if rank in ranks}
        dead = set()
        for ins in prog.for_rank(rank):
            if isinstance(ins, Delete):
                for v in ins.vids:
                    live.discard(v)
                    dead.add(v)
                continue
            uses, defs = _uses_defs(ins, rank)
            for v in uses:
                if v in dead and v not in live:
                    raise ProgramError(f"rank {rank}: %{v} used after delete by {ins}")
                if v not in live:
                    raise ProgramError(f"rank {rank}: %{v} used before definition by {ins}")
            for v in defs:
                live.add(v)
                dead.discard(v)
        for o in prog.outputs:
            if o[0] == "v" and rank in o[2] and o[1] not in live:
                raise ProgramError(f"rank {rank}: output %{o[1]} is not live at the end of the program")

    # ---- transfer / collective bookkeeping ------------------------------------------------------------
    tids = [i.tid for i in prog.instrs if isinstance(i, Transfer)]
    if len(set(tids)) != len(tids) or tids != sorted(tids):
        raise ProgramError("transfer ids must be unique and increasing in program order")
    joined = defaultdict(set)
    for i in prog.instrs:
        if isinstance(i, (AllReduce, AllGather)):
            joined[i.cid].add(i.rank)
    for i in prog.instrs:
        if isinstance(i, (AllReduce, AllGather)) and joined[i.cid] != set(i.ranks):
            raise ProgramError(f"collective #{i.cid} joined by {sorted(joined[i.cid])}, expected {i.ranks}")

    # ---- deadlock replay with rendezvous semantics -----------------------------------------------------
    progs = [prog.for_rank(r) for r in range(prog.n_ranks)]
    pc = [0] * prog.n_ranks
    steps = 0
    while True:
        progressed = False
        for r in range(prog.n_ranks):
            while pc[r] < len(progs[r]):
                ins = progs[r][pc[r]]
                if isinstance(ins, Transfer):
                    other = ins.dst if ins.rank == r else ins.rank
                    # rendezvous: the peer's next communication instruction must be this transfer
                    if pc[other] < len(progs[other]) and progs[other][pc[other]] is ins:
                        pc[r] += 1
                        pc[other] += 1
                        progressed = True
                        continue
                    break
                if isinstance(ins, (AllReduce, AllGather)):
                    peers = ins.ranks
                    at = []
                    for p in peers:
                        nxt = progs[p][pc[p]] if pc[p] < len(progs[p]) else None
                        at.append(isinstance(nxt, (AllReduce, AllGather)) and nxt.cid == ins.cid)
                    if all(at):
                        for p in peers:
                            pc[p] += 1
                        progressed = True
                        continue
                    break
                pc[r] += 1
                progressed = True
        if all(pc[r] == len(progs[r]) for r in range(prog.n_ranks)):
            break
        if not progressed:
            where = {r: str(progs[r][pc[r]]) for r in range(prog.n_ranks) if pc[r] < len(progs[r])}
            raise ProgramError(f"per-rank programs deadlock under blocking point-to-point semantics at {where}")
        steps += 1
    return {"replay_rounds": steps, "n_transfers": len(tids)}
