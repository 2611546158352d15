"""TEST INFRASTRUCTURE (never on a product path): a numpy restatement of the expert-parallel token exchange's
bookkeeping — which place of which owner's receive region a routed pair goes to, the words that travel with it,
and the way home.  There is no counterpart in the reference (its experts all live on one device,
src/weights.rs:55-58); what the exchange must preserve is the single-device layer (Generic::moe,
src/generic.rs:508-574): every pair run on its expert, the rows summed with the router's weights in route order.
Parity for this file is therefore pinned by construction against oracle.moe_sum / oracle.route, not by a
reference vector."""
import numpy as np

ROUTE_SKIP = 0xFFFFFFFF


def dispatch_plan(ids, world: int, experts_per_rank: int, cap: int):
    """Where the pairs of one sending rank go.  `ids`: its global expert ids in route order.  Returns
    (owner[pairs], place[pairs], meta[world][cap]) — place = number of earlier pairs of the same owner; meta of
    a used place = local expert id | pair index << 16, of an unused one ROUTE_SKIP."""
    ids = np.asarray(ids, dtype=np.int64).reshape(-1)
    assert len(ids) <= cap and len(ids) < 65536 and experts_per_rank <= 65536
    owner = ids // experts_per_rank
    assert owner.max(initial=0) < world
    place = np.zeros(len(ids), dtype=np.int64)
    seen = np.zeros(world, dtype=np.int64)
    meta = np.full((world, cap), ROUTE_SKIP, dtype=np.uint32)
    for p, (e, o) in enumerate(zip(ids, owner)):
        place[p] = seen[o]
        meta[o, seen[o]] = np.uint32((e - o * experts_per_rank) | (p << 16))
        seen[o] += 1
    return owner, place, meta


def receive_regions(metas, rank: int):
    """The receive area of `rank`: region s = what rank s's plan holds for this owner.  `metas`: the meta
    tables of all sending ranks, in rank order.  Returns meta[world * cap] and the ids the routed projections
    get (local expert id or ROUTE_SKIP)."""
    region = np.concatenate([np.asarray(m)[rank] for m in metas]).astype(np.uint32)
    ids = np.where(region == ROUTE_SKIP, np.uint32(ROUTE_SKIP), region & np.uint32(0xFFFF)).astype(np.uint32)
    return region, ids


def way_home(region, cap: int):
    """For every live place of a receive area: (place, home rank, pair index at home)."""
    region = np.asarray(region, dtype=np.uint32)
    live = np.nonzero(region != ROUTE_SKIP)[0]
    return [(int(i), int(i // cap), int(region[i] >> 16)) for i in live]
