"""``Rki4State`` -- every persistent buffer of the page selector, allocated once.

Same constructor, attribute names and per-step scratch as the reference's
``selection/rki4_state.py:157-354``.  The seven summary components of a
(physical block, kv-head) live in ONE 832-byte record so that the scorer can
fetch a page summary with a single contiguous bulk copy; ``pp_v4``, ``pp_vs``,
``pp_c8``, ``pp_cs``, ``pp_mu8`` and ``pp_mus`` are strided views into
``pp_rec`` with the reference's shapes and dtypes (the reference has the same
arrangement behind its ``RKI4_MMA_AOS`` switch, lines 93-102 and 198-220).

HBM layout, per layer: ``pp_rec (NB, n_kv, 832) u8`` + ``pp_tag (NB, n_kv, 8)
bf16`` = 848 B per (block, kv-head), i.e. ~10 % of the 8 KiB bf16 K+V page.
"""
from __future__ import annotations

import torch

TAGW = 8
RNK = 8
IBITS = 4
QMAX, QMIN = 7, -8
REC_BYTES = 832

# byte offsets of the record fields (mirrored in csrc/common.cuh)
RO_V4, RO_MU8, RO_C8, RO_CS, RO_VS, RO_MUS = 0, 512, 640, 768, 800, 816


def record_bytes(d: int, page: int, tagw: int = TAGW) -> int:
    """Footprint of one (block, kv-head) summary INCLUDING the tag
    (reference ``record_bytes``, lines 124-141, in its record mode)."""
    if d != 128 or page != 16:
        raise AssertionError("summary records cover head_dim 128 / page 16 only")
    return REC_BYTES + 2 * tagw


class Rki4State:
    """Summary slabs + per-step selection outputs for one engine.

    Every tensor address is stable for the life of the object, so the scoring,
    selection and decode launches can be captured in a CUDA graph.
    """

    def __init__(self, device, *, num_layers: int, num_blocks: int, n_kv: int,
                 G: int, head_dim: int, page: int, max_reqs: int,
                 max_pages: int, rank: int = RNK, budget: float = 0.1,
                 budget_pages=None, sink_pages: int = 1, window_pages: int = 1,
                 tagw: int = TAGW, combine: str = "nrm", zsplit=None):
        assert window_pages >= 1, \
            "window_pages >= 1: the partial tail page must sit inside the window"
        self.validate_geometry(head_dim=head_dim, G=G, page=page, rank=rank)
        assert combine in ("max", "nrm")
        assert zsplit is None or zsplit >= 1, \
            f"zsplit must be None (auto) or >= 1, got {zsplit}"
        assert tagw == TAGW, f"tag width is fixed at {TAGW}"
        L, NB, D, MP, R = num_layers, num_blocks, head_dim, max_pages, max_reqs
        self.L, self.NB, self.n_kv, self.G, self.d = L, NB, n_kv, G, D
        self.D = D
        self.page, self.r, self.tagw = page, RNK, tagw
        self.v_bits = IBITS
        self.max_reqs, self.max_pages = R, MP
        self.budget = float(budget)
        self.budget_abs = int(budget_pages or 0)
        self.sink_pages, self.window_pages = int(sink_pages), int(window_pages)
        self.combine = combine
        self.zsplit = int(zsplit) if zsplit else None
        self.device = device
        u8, i8, bf16 = torch.uint8, torch.int8, torch.bfloat16
        i32, f32, f64 = torch.int32, torch.float32, torch.float64

        # ---- summaries: one record per (layer, block, kv-head) ---------------
        self.pp_rec = torch.zeros(L, NB, n_kv, REC_BYTES, device=device, dtype=u8)
        rec = self.pp_rec
        self.pp_v4 = rec[..., RO_V4:RO_MU8].unflatten(-1, (RNK, D // 2))
        self.pp_mu8 = rec[..., RO_MU8:RO_C8].view(i8)
        self.pp_c8 = rec[..., RO_C8:RO_CS].view(i8).unflatten(-1, (page, RNK))
        self.pp_cs = rec[..., RO_CS:RO_VS].view(bf16)
        self.pp_vs = rec[..., RO_VS:RO_MUS].view(bf16)
        self.pp_mus = rec[..., RO_MUS:RO_MUS + 2].view(bf16).squeeze(-1)
        # NaN never equals anything: every page is stale until first built
        self.pp_tag = torch.full((L, NB, n_kv, tagw), float("nan"),
                                 device=device, dtype=bf16)

        # ---- per-step outputs (request-row keyed) ----------------------------
        self.score = torch.zeros(R, n_kv, MP, device=device, dtype=f32)
        self.page_table = torch.full((R, n_kv, MP), -1, device=device, dtype=i32)
        self.page_cnt = torch.zeros(R, n_kv, device=device, dtype=i32)
        self.score_h = torch.zeros(R, n_kv, G, MP, device=device, dtype=f32)
        # per-head score maxima as order-preserving uint32 keys; 0 = "unset"
        self.hmax = (torch.zeros(R, n_kv, G, device=device, dtype=i32)
                     if combine == "nrm" else None)
        self.n_pages = torch.zeros(R, device=device, dtype=i32)
        self.n_sel_hi = torch.zeros(R, device=device, dtype=i32)
        self.b_fix = torch.ones(R, device=device, dtype=i32)
        self.budget64 = torch.tensor([self.budget], device=device, dtype=f64)
        # optional per-request page budgets (see set_request_budgets)
        self.budget_req = None
        # device word a kernel raises when one of its bounded waits runs out
        self.status = torch.zeros(1, device=device, dtype=i32)

        # split-K partials are attached by attention.ensure_stage_b_buffers
        self.m_part = self.l_part = self.acc_part = None
        self.split = None
        self.scale = None
        self._k_ptrs = None
        self._k_ptrs_key = None

        planned = record_bytes(D, page, tagw) * n_kv * NB
        assert self.bytes_per_layer() == planned

    @staticmethod
    def validate_geometry(*, head_dim: int, G: int, page: int,
                          rank: int = RNK) -> None:
        """Supported set of this build, checked at wiring time so that an
        unsupported model fails before any kernel runs (reference lines
        288-334; the reference admits d in {64,128,256}, page in {16,32,64}
        and G <= 8 -- here head_dim 128, page 16, and G up to 16)."""
        assert head_dim == 128, \
            f"rki4 (B200 build) supports head_dim 128, model has d={head_dim}"
        assert 1 <= G <= 16, \
            f"rki4 (B200 build) supports 1 <= G <= 16 query heads per kv head, got G={G}"
        assert page == 16, \
            f"rki4 (B200 build) supports block_size 16, engine block_size={page}"
        assert rank == RNK, f"rki4 rank is fixed at {RNK}, got rank={rank}"

    @classmethod
    def record_bytes(cls, d: int, page: int, tagw: int = TAGW) -> int:
        return record_bytes(d, page, tagw)

    def bytes_per_layer(self) -> int:
        return self.pp_rec[0].numel() + self.pp_tag[0].numel() * 2

    def layer_state(self, layer: int):
        """(v4, vs, c8, cs, mu8, mus, tag) views of one layer."""
        return (self.pp_v4[layer], self.pp_vs[layer], self.pp_c8[layer],
                self.pp_cs[layer], self.pp_mu8[layer], self.pp_mus[layer],
                self.pp_tag[layer])

    def set_request_budgets(self, budget_pages) -> None:
        """One page budget per request row (a continuous batch whose requests
        carry their own budgets): ``derive_page_params`` then takes ``b_fix[r]``
        from ``budget_pages[r]`` (> 0: pages, <= 0: the fraction ``budget``)
        instead of the engine-wide ``budget_pages``.  ``None`` switches back.
        The reference holds ``b_fix`` per request but fills it from one
        constant (``selection/select.py:29-58``)."""
        if budget_pages is None:
            self.budget_req = None
            return
        b = torch.as_tensor(budget_pages, dtype=torch.int32).reshape(-1)
        assert b.numel() <= self.max_reqs
        if self.budget_req is None:
            self.budget_req = torch.zeros(self.max_reqs, device=self.device,
                                          dtype=torch.int32)
        self.budget_req.zero_()
        self.budget_req[:b.numel()].copy_(b)

    def check_status(self) -> None:
        """Host-side read of the kernel status word (synchronises)."""
        s = int(self.status.item())
        if s != 0:
            self.status.zero_()
            raise RuntimeError(f"a LOCKS kernel reported status {s} "
                               "(1 = an on-chip wait timed out)")
