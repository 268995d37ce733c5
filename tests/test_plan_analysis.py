"""Which recorded operators may share one resident launch, and how their reads and writes are
resolved: the rule of nn_plan_end, exercised on address ranges alone (no GPU).

The step mirrors the reference's decode loop (src/models/smollm2-135m-instruct/src/model.cpp:
88-239): per layer QKV, o_proj + residual, gate/up/SiLU, down + residual, then lm_head."""
import ctypes

import numpy as np
import pytest


class Ops:
    """A list of operators given by the address ranges they touch."""

    def __init__(self):
        self.rows = []

    def add(self, x, x_bytes, outs, inplace=False, argmax=False):
        self.rows.append((x, x_bytes, list(outs), inplace, argmax))
        return len(self.rows) - 1

    def analyze(self, L, first=0):
        n = len(self.rows)
        xa = np.array([r[0] for r in self.rows], np.uint64)
        xb = np.array([r[1] for r in self.rows], np.uint64)
        oa = np.zeros((n, 4), np.uint64)
        ob = np.zeros((n, 4), np.uint64)
        no = np.zeros(n, np.int32)
        fl = np.zeros(n, np.int32)
        for i, (_, _, outs, inplace, argmax) in enumerate(self.rows):
            no[i] = len(outs)
            for k, (a, b) in enumerate(outs):
                oa[i, k], ob[i, k] = a, b
            fl[i] = (1 if inplace else 0) | (2 if argmax else 0)
        xd, rd, sm, pm = (np.full(n, -9, np.int32) for _ in range(4))
        p = lambda a: a.ctypes.data_as(ctypes.c_void_p)
        length = L.nn_plan_analyze(n, p(xa), p(xb), p(oa), p(ob), p(no), p(fl), first, p(xd), p(rd), p(sm), p(pm))
        return length, xd[:max(length, 0)], rd[:max(length, 0)], sm[:max(length, 0)], pm[:max(length, 0)]


H, Q, KV, F, V = 576, 576, 192, 1536, 49152
RES, XH, XATT, XACT, QB, KB, VB, ACT, LOG, TOK = (0x100000 * (i + 1) for i in range(10))


def step(layers, chained):
    """chained: every projection reads what the step itself produced (the residual stream, q, the
    SwiGLU output); otherwise each reads a fixed buffer, as a caller does whose own kernels
    (norms, attention) sit between the projections."""
    o = Ops()
    for _ in range(layers):
        o.add(RES if chained else XH, 2 * H, [(QB, 2 * Q), (KB, 2 * KV), (VB, 2 * KV)])
        o.add(QB if chained else XATT, 2 * Q, [(RES, 2 * H)], inplace=True)
        o.add(RES if chained else XH, 2 * H, [(ACT, 2 * F)])
        o.add(ACT if chained else XACT, 2 * F, [(RES, 2 * H)], inplace=True)
    o.add(RES if chained else XH, 2 * H, [(LOG, 2 * V), (TOK, 4)], argmax=True)
    return o


def test_chained_step_is_one_run(built_lib):
    L = built_lib
    layers = 3
    n, xd, rd, sm, pm = step(layers, True).analyze(L)
    assert n == 4 * layers + 1
    for l in range(layers):
        q, o, g, d = 4 * l, 4 * l + 1, 4 * l + 2, 4 * l + 3
        assert xd[q] == (d - 4 if l else -1)          # the residual stream of the previous layer
        assert xd[o] == q and xd[g] == o and xd[d] == g
        assert rd[o] == (d - 4 if l else -1) and rd[d] == o   # each in-place add updates the previous add's values
        last = l == layers - 1
        assert sm[q] == (0b111 if last else 0)        # q, k, v are overwritten by the next layer's QKV
        assert pm[q] == 0b001                         # only q is read inside the run
        assert sm[o] == 0 and pm[o] == 1              # the down projection overwrites the residual stream
        assert sm[g] == (1 if last else 0) and pm[g] == 1
        assert sm[d] == (1 if last else 0) and pm[d] == 1
    assert xd[-1] == 4 * layers - 1 and sm[-1] == 1 and pm[-1] == 0


def test_fixed_inputs_are_one_run_with_row_wise_residual_chain(built_lib):
    n, xd, rd, sm, pm = step(2, False).analyze(built_lib)
    assert n == 9
    assert (xd == -1).all()                           # every x was written before the run
    assert list(rd[[1, 3, 5, 7]]) == [-1, 1, 3, 5]    # in-place adds follow one another row by row
    assert list(sm[[1, 3, 5, 7]]) == [0, 0, 0, 1]
    assert list(pm[[1, 3, 5]]) == [1, 1, 1] and pm[7] == 0


def test_reader_of_old_contents_not_ordered_before_an_overwrite_ends_the_run(built_lib):
    o = Ops()
    o.add(RES, 2 * H, [(QB, 2 * Q)])                  # reads the residual stream as it was before the run
    o.add(XATT, 2 * Q, [(RES, 2 * H)], inplace=True)  # overwrites it, and nothing orders it behind that read
    n, *_ = o.analyze(built_lib)
    assert n == 1
    # with the overwrite consuming the reader's output, the data flow orders them
    o = Ops()
    o.add(RES, 2 * H, [(QB, 2 * Q)])
    o.add(QB, 2 * Q, [(RES, 2 * H)], inplace=True)
    n, xd, rd, sm, pm = o.analyze(built_lib)
    assert n == 2 and xd[1] == 0 and rd[1] == -1 and pm[0] == 1


def test_partial_and_straddling_reads_end_the_run(built_lib):
    o = Ops()
    o.add(XH, 2 * H, [(QB, 2 * Q)])
    o.add(QB, Q, [(ACT, 2 * F)])                      # half of q
    assert o.analyze(built_lib)[0] == 1
    o = Ops()
    o.add(XH, 2 * H, [(QB, 2 * Q), (QB + 2 * Q, 2 * KV)])
    o.add(QB, 2 * Q + 2 * KV, [(ACT, 2 * F)])          # q and k as one vector
    assert o.analyze(built_lib)[0] == 1
    o = Ops()
    o.add(XH, 2 * H, [(XH, 2 * H)])                    # in place on its own input
    assert o.analyze(built_lib)[0] == 0
    o = Ops()
    o.add(XH, 2 * H, [(QB, 2 * Q)])
    o.add(XATT, 2 * Q, [(QB + 64, 2 * Q)])             # overlaps an earlier output without matching it
    assert o.analyze(built_lib)[0] == 1


def test_non_inplace_overwrite_after_an_inplace_reader_of_old_rows_needs_the_chain(built_lib):
    o = Ops()
    o.add(XATT, 2 * Q, [(RES, 2 * H)], inplace=True)   # reads the old rows of RES
    o.add(XH, 2 * H, [(RES, 2 * H)])                   # plain overwrite, unrelated input: unordered
    assert o.analyze(built_lib)[0] == 1
    o = Ops()
    a = o.add(XATT, 2 * Q, [(RES, 2 * H)], inplace=True)
    o.add(RES, 2 * H, [(ACT, 2 * F)])
    o.add(ACT, 2 * F, [(RES, 2 * H)])                  # plain overwrite fed by the chain behind the reader
    n, xd, rd, sm, pm = o.analyze(built_lib)
    assert n == 3 and sm[a] == 0 and rd[2] == -1


def test_one_greedy_pick_per_run_and_start_offset(built_lib):
    o = Ops()
    o.add(XH, 2 * H, [(LOG, 2 * V), (TOK, 4)], argmax=True)
    o.add(XH, 2 * H, [(LOG + 0x40000, 2 * V), (TOK + 64, 4)], argmax=True)
    assert o.analyze(built_lib)[0] == 1
    # analysis from an offset numbers the operators relative to it
    s = step(2, True)
    n, xd, rd, sm, pm = s.analyze(built_lib, first=4)
    assert n == 5 and xd[0] == -1 and xd[1] == 0 and rd[1] == -1 and rd[3] == 1
    assert s.analyze(built_lib, first=9)[0] == 0
    assert built_lib.nn_plan_analyze(-1, None, None, None, None, None, None, 0, None, None, None, None) < 0
