"""Generates tile_table.h: the (dimension, degree, chain length, group) variants of the
register-tile kernels that are compiled into libcusig.so.

Run by hand after changing the heuristics:  python pysiglib_b200/csrc/gen_tile_table.py

For every covered (augmented dimension D, degree N) and dtype the table holds up to three
variants per direction:
  * "big":   the largest tile that fits the register budget (least redundant chain work);
  * "mid" / "small": tiles with at least 2x / 4x as many execution units per path, chosen
             at run time when the batch alone does not give enough warps to fill the GPU.
"""
import os

# (D, max degree) pairs covered by the tile kernels with up to three tile sizes each; everything
# else runs on the generic kernels
COVER = {2: 12, 3: 9, 4: 8, 5: 7, 6: 6, 7: 5, 8: 5, 9: 5, 10: 5, 11: 4, 12: 4, 13: 4, 14: 4, 15: 4,
         16: 4, 17: 4, 20: 3, 24: 3, 32: 3, 33: 3}
# Deeper degrees, one tile size each (the biggest): long chains (P up to N - 2) over many units per
# path.  These are the shapes the reference serves with its register "Tree" kernels
# (siglib/cusig/cu_signature_horner.cuh:267-307, 389-438: d = 6 up to degree 9, and in float64
# d = 8, 10, 12, 16, 24, 32 up to degree 8 where the signature still fits 2^31 coefficients), plus the
# benchmark shapes after time augmentation / lead-lag (d' = 4 at degree 12, 10 and 11 at degree 7 / 5,
# 20 and 21 at degree 5, 32 and 33 at degree 4).
DEEP = {4: 12, 6: 9, 7: 6, 8: 8, 9: 6, 10: 8, 11: 5, 12: 8, 16: 7, 20: 5, 21: 5, 24: 6, 32: 6, 33: 4}
MAX_UNITS = 1 << 24  # execution units (threads) per path
# register budget in tile values per unit: (forward, backward) by dtype.  The backward keeps the
# whole adjoint tile but no level-N state, so its budget is close to the forward one.
BUDGET = {"float": (160, 136), "double": (72, 72)}
PARTS = 24


def geom(d, k):
    return sum(d ** i for i in range(k))


def fwd_instr(D, N, P, G):
    """Issue slots of one forward step of one unit (same counting as tile_math.h: tile_update)."""
    Q = N - P
    nodes = lambda q: G * D ** (q - 1)
    n = 0
    for t in range(1, Q + 1):
        n += 3 * P + 1
        if t == 1:
            n += G
        else:
            n += 1 + G
            for q in range(2, t):
                n += nodes(q - 1) * (2 + D)
            n += nodes(t - 1) * (1 + D)
    for T in range(1, P + 1):
        n += 3 * (T - 1) + 2
    return n + (D + 3) // 4 + (G + 3) // 4 + P + 4


def bwd_instr(D, N, P, G):
    """Rewind + pull-back (about twice the forward tile work) + the warp reduction."""
    dp2 = 1
    while dp2 < D:
        dp2 *= 2
    return 3 * fwd_instr(D, N, P, G) + 4 * dp2 + D + 12 * P + 20


def variants(D, N, budget):
    cands = []
    for P in range(0, N):
        for G in [g for g in range(1, D + 1) if D % g == 0]:
            ts = G * geom(D, N - P)
            units = D ** P * (D // G)
            if ts <= budget and units <= MAX_UNITS:
                cands.append((ts, units, P, G))
    if not cands:
        return []
    full = [c for c in cands if c[1] >= 32]
    # biggest tile among those filling a warp; else the tile with most units
    big = max(full, key=lambda c: (c[0], -c[2])) if full else max(cands, key=lambda c: (c[1], c[0]))
    out = [big]
    for mult in (2, 4):
        more = [c for c in cands if c[1] >= mult * big[1] and c[0] >= 8 and c not in out]
        if more:
            pick = max(more, key=lambda c: (c[0], -c[2]))
            if pick[0] < out[-1][0]:
                out.append(pick)
    return out


def emit(path, parts_n, only=None):
    """Writes the table header.  only: a set of (D, N) pairs to restrict the table to (a library for
    a fixed set of shapes builds in a fraction of the time), None for every covered shape."""
    entries = []  # (cost, text)
    for tname, (bf, bb) in BUDGET.items():
        for D in sorted(set(COVER) | set(DEEP)):
            for N in range(2, max(COVER.get(D, 0), DEEP.get(D, 0)) + 1):
                if only is not None and (D, N) not in only:
                    continue
                if D ** N >= 1 << 31:
                    continue
                deep = N > COVER.get(D, 0)
                for backward, budget in ((0, bf), (1, bb)):
                    for rank, (ts, units, P, G) in enumerate(variants(D, N, budget)[:1 if deep else 3]):
                        # the biggest forward tile of a shape also gets the fused log-signature sweep
                        # (where a path fits a portable cluster of 8 CTAs of 4 warps and the shared copy of
                        # the levels below N stays under 96 KB)
                        # and the tile is shallow: at most 16 rows of level-N coefficients per unit)
                        rows = 1 if N - P < 2 else G * D ** (N - P - 2)
                        fits = (units <= 1024 and geom(D, N) * (8 if tname == "double" else 4) <= 96 * 1024
                                and N - P <= 3 and rows <= 16)
                        log = 1 if (not backward and rank == 0 and fits) else 0
                        cost = ts * (3 if backward else (2 if log else 1))
                        est = bwd_instr(D, N, P, G) if backward else fwd_instr(D, N, P, G)
                        entries.append((cost, "X(%s, %d, %d, %d, %d, %d, %d, %d)" % (tname, backward, D, N, P, G, est, log)))
    entries.sort(key=lambda e: -e[0])
    parts = [[] for _ in range(parts_n)]
    loads = [0] * parts_n
    for cost, text in entries:
        i = loads.index(min(loads))
        parts[i].append(text)
        loads[i] += cost
    with open(path, "w") as f:
        f.write("// Generated by gen_tile_table.py; do not edit by hand.\n")
        f.write("// X(type, backward, D, N, P, G, est, log): one compiled register-tile kernel variant; est = estimated\n// issue slots per unit and step (cost model of the run-time variant choice); log = 1: the fused\n// log-signature sweep is compiled for it too.\n")
        f.write("#pragma once\n#define SIG_TILE_PARTS %d\n" % parts_n)
        f.write("#define SIG_TILE_PART_LIST(F) " + " ".join("F(%d)" % i for i in range(parts_n)) + "\n")
        for i, part in enumerate(parts):
            f.write("#define SIG_TILE_PART_%d(X) \\\n" % i)
            f.write(" \\\n".join("    " + t for t in sorted(part)) + "\n")
    print(path, len(entries), "variants in", parts_n, "parts; loads", loads)


def main():
    here = os.path.dirname(os.path.abspath(__file__))
    emit(os.path.join(here, "tile_table.h"), PARTS)


if __name__ == "__main__":
    main()
