"""TEST INFRASTRUCTURE — plain-torch CPU restatements of the kernel primitives (not shipped).

:class:`OracleBackend` has the same methods as ``mlcg_b200.backend.CudaBackend``.  The test-suite uses
it in two ways: as the checker the CUDA kernels are compared against (same inputs, ``-m gpu``), and,
substituted by the tests' ``monkeypatch`` fixture for the package's back-end object, to exercise the host-side autograd wiring on a
machine without a GPU.  It is never selected by the package itself.
"""
import numpy as np
import torch

from . import radius_ref, schnet_ref


def _expand_segments(ptr):
    counts = (ptr[1:] - ptr[:-1]).to(torch.int64)
    return torch.repeat_interleave(torch.arange(counts.numel(), device=ptr.device), counts)


class OracleBackend:
    name = "oracle"

    # ------------------------------------------------------------------ radius graph
    def batch_to_ptr(self, batch, B):
        return torch.from_numpy(radius_ref.batch_to_ptr(batch.cpu().numpy(), B)).to(batch.device)

    def radius_graph(self, pos, ptr, r, max_num_neighbors, loop, rule, want_distance=False, want_batch=True, exclude=None):
        p = pos.detach().cpu().numpy()
        rule_name = "cluster" if int(rule) == 1 else "native"
        N = p.shape[0]
        if exclude is None:
            graph = lambda cap, **kw: radius_ref.radius_graph_c(p, ptr.cpu().numpy(), r, cap, loop, rule_name, **kw)
        else:
            ex = tuple(t.cpu().numpy() for t in exclude)
            graph = lambda cap, **kw: radius_ref.radius_graph_numpy(p, ptr.cpu().numpy(), r, cap, loop, rule_name, exclude=ex, **kw)
        ei, dist = graph(max_num_neighbors, with_distance=True)
        deg = np.bincount(ei[0], minlength=N)
        offsets = np.zeros(N + 1, dtype=np.int64)
        np.cumsum(deg, out=offsets[1:])
        # truncated: any centre that would have had more neighbours without the cap
        full = graph(max(N, 1) + 1)
        status = 1 if full.shape[1] != ei.shape[1] else 0
        dev = pos.device
        ei_t = torch.from_numpy(ei).to(dev)
        seg = torch.from_numpy(np.searchsorted(ptr.cpu().numpy(), ei[0], side="right") - 1).to(dev)
        return dict(edge_index=ei_t, distance=torch.from_numpy(dist).to(dev) if want_distance else None,
                    mapping_batch=seg if want_batch else None, row0=ei_t[0].to(torch.int32), row1=ei_t[1].to(torch.int32),
                    offsets=torch.from_numpy(offsets).to(dev), status=status)

    def radius_graph_pbc(self, pos, ptr, cells, repeats, r, max_num_neighbors, loop, want_distance=False, want_batch=True):
        p, pt = pos.detach().cpu().numpy(), ptr.cpu().numpy()
        # `repeats` already holds the copies per direction: a direction is periodic exactly where it is non-zero or r allows none
        ei, shifts = radius_ref.radius_graph_pbc_numpy(p, pt, cells.detach().cpu().numpy(), repeats.cpu().numpy() > 0, r, max_num_neighbors, loop)
        dev = pos.device
        ei_t, sh = torch.from_numpy(ei).to(dev), torch.from_numpy(shifts).to(dev)
        dist = ((pos[ei_t[1]] + sh) - pos[ei_t[0]]).norm(dim=1).detach() if want_distance else None
        seg = torch.from_numpy(np.searchsorted(pt, ei[0], side="right") - 1).to(dev)
        return dict(edge_index=ei_t, cell_shifts=sh, distance=dist, mapping_batch=seg if want_batch else None, status=0)

    def edge_twin(self, row0, row1, offsets, N, fresh_status=False):
        E = row0.numel()
        key = row0.to(torch.int64) * N + row1.to(torch.int64)
        rkey = row1.to(torch.int64) * N + row0.to(torch.int64)
        pos = torch.searchsorted(key, rkey).clamp(max=max(E - 1, 0))
        found = key[pos] == rkey if E else torch.zeros(0, dtype=torch.bool)
        twin = torch.where(found, pos, torch.full_like(pos, -1)).to(torch.int32)
        status = torch.zeros(4, dtype=torch.int32)
        if E and not bool(found.all()):
            status[0] = 4
        return twin, status

    def check_pending(self):
        pass            # the restatements report nothing lazily

    def pair_plan(self, row0, row1, offsets, N, fresh_status=False):
        twin, status = self.edge_twin(row0, row1, offsets, N)
        sel = torch.nonzero(row0 < row1).flatten().to(torch.int32)
        return twin, sel, self.pair_index(sel, twin), status

    def pair_index(self, sel, twin):
        pair_of = torch.full((twin.numel(),), -1, dtype=torch.int32)
        k = torch.arange(sel.numel(), dtype=torch.int32)
        pair_of[sel.long()] = k
        pair_of[twin[sel.long()].long()] = k
        return pair_of

    # ------------------------------------------------------------------ geometry
    def edge_diff(self, pos, row0, row1):
        return pos[row1.long()] - pos[row0.long()]

    def edge_distance(self, pos, row0, row1):
        return (pos[row1.long()] - pos[row0.long()]).norm(p=2, dim=1)

    def edge_distance_backward(self, pos, g, d, plan):
        w = (g / d).unsqueeze(-1) * (pos[plan.row1.long()] - pos[plan.row0.long()])
        return self.node_scatter_diff(w, plan.ptr_in, plan.perm_in, plan.ptr_out, plan.perm_out, plan.N)

    def node_scatter_diff(self, g, ptr_in, perm_in, ptr_out, perm_out, N):
        gi = g if perm_in is None else g[perm_in.long()]
        go = g if perm_out is None else g[perm_out.long()]
        out = torch.zeros((N, 3), dtype=g.dtype)
        out.index_add_(0, _expand_segments(ptr_in), gi)
        out.index_add_(0, _expand_segments(ptr_out), -go)
        return out

    # ------------------------------------------------------------------ radial basis
    @staticmethod
    def _phi(d, spec, keep_graph=False):
        cut = {"cutoff": "cosine" if spec.cutoff_kind == 1 else "identity", "lower": spec.lower, "upper": spec.upper}
        s = {"kind": "gaussian" if spec.kind == 0 else "expnormal", "rbf_cutoff": cut}
        p0, p1 = (spec.p0, spec.p1) if keep_graph else (spec.p0.detach(), spec.p1.detach())
        sd = {"rbf_layer.offset": p0.to(d.dtype), "rbf_layer.coeff": p1.to(d.dtype).reshape(-1)[0],
              "rbf_layer.means": p0.to(d.dtype), "rbf_layer.betas": p1.to(d.dtype).reshape(-1)}
        return schnet_ref.radial_basis(d, s, sd)

    def rbf_expand(self, d, spec, order):
        """order-th derivative by nested automatic differentiation of the oracle expression."""
        d = d.detach().clone().requires_grad_(True)
        with torch.enable_grad():
            cur = self._phi(d, spec)
            for _ in range(order):
                cols = [torch.autograd.grad(cur[:, k].sum(), d, create_graph=True)[0] for k in range(cur.shape[1])]
                cur = torch.stack(cols, dim=1)
        return cur.detach()

    def rbf_contract(self, d, G, spec, order):
        return (G.detach() * self.rbf_expand(d, spec, order)).sum(dim=1)

    def rbf_param_contract(self, d, G, c, spec, order):
        """Gradients of sum_e c[e] sum_k G[e,k] phi_k^(order)(d_e) with respect to the basis' two parameter tensors, by
        automatic differentiation of the oracle expression."""
        import dataclasses
        sp = dataclasses.replace(spec, p0=spec.p0.detach().clone().requires_grad_(True), p1=spec.p1.detach().clone().requires_grad_(True))
        dd = d.detach().clone().requires_grad_(True)
        with torch.enable_grad():
            cur = self._phi(dd, sp, keep_graph=True)
            for _ in range(order):
                cols = [torch.autograd.grad(cur[:, k].sum(), dd, create_graph=True)[0] for k in range(cur.shape[1])]
                cur = torch.stack(cols, dim=1)
            w = G.detach() if c is None else G.detach() * c.detach().unsqueeze(-1)
            gp0, gp1 = torch.autograd.grad((w * cur).sum(), [sp.p0, sp.p1])
        return gp0.reshape(-1), gp1.reshape(-1)

    # ------------------------------------------------------------------ CFConv primitives
    def seg_mul_sum(self, a, V, ptr, nbr, eperm, N):
        Vp = V if eperm is None else V[eperm.long()]
        out = torch.zeros((N, V.shape[1]), dtype=V.dtype)
        return out.index_add_(0, _expand_segments(ptr), a[nbr.long()] * Vp)

    def edge_mul(self, a, b, ia, ib):
        return a[ia.long()] * b[ib.long()]

    def pair_mul(self, a, b, ia, ib):
        return a[ia.long()] * b[ib.long()] + a[ib.long()] * b[ia.long()]

    def gemm_tn_colsum(self, G, X):
        return G.t() @ X, G.sum(0)

    def tanh_grad(self, mode, G, g, y):
        return g * (1 - y * y) if mode == 0 else -2 * G * g * y

    def row_scale(self, a, c):
        return a * c.unsqueeze(-1)

    def row_dot(self, a, b):
        return (a * b).sum(dim=1)

    def gemm(self, mode, A, B, bias=None):
        if mode == 0:
            C = A @ B.t()
            return C + bias if bias is not None else C
        if mode == 1:
            return A @ B
        return A.t() @ B

    def segment_sum(self, x, ptr):
        out = torch.zeros(ptr.numel() - 1, dtype=x.dtype)
        return out.index_add_(0, _expand_segments(ptr), x)

    # ------------------------------------------------------------------ Langevin integrator (langevin.py:100-144)
    def langevin_first_half(self, x, v, f, masses, beta_mass_ratio, noise, dt, vscale, noisescale):
        vn = v + 0.5 * dt * f / masses[:, None]
        xn = x + vn * dt * 0.5
        vn = vn * vscale + noisescale * (beta_mass_ratio[:, None] * noise)
        xn = xn + vn * dt * 0.5
        x.copy_(xn)
        v.copy_(vn)

    def langevin_second_half(self, v, f, masses, dt):
        v.copy_(v + 0.5 * dt * f / masses[:, None])

    # ------------------------------------------------------------------ priors
    def prior_terms(self, kind, pos, mapping, mapping_batch, params, B, want_grad=True):
        p = pos.detach().clone().requires_grad_(True)
        with torch.enable_grad():
            if kind == 0:
                y = params[1] * (schnet_ref.edge_distances(p, mapping) - params[0]) ** 2
            elif kind == 1:
                y = params[1] * (schnet_ref.angles_cos(p, mapping) - params[0]) ** 2
            elif kind == 2:
                n = (params.shape[0] - 1) // 2
                th = schnet_ref.torsions(p, mapping)
                y = params[0].clone()
                for i in range(1, n + 1):
                    y = y + params[i] * torch.sin(i * th) + params[n + i] * torch.cos(i * th)
            else:
                rr = (params[0] / schnet_ref.edge_distances(p, mapping)) ** 2
                y = rr * rr * rr
            e = schnet_ref.index_sum(y, mapping_batch, B)
            g = torch.autograd.grad(e.sum(), p)[0] if want_grad else None
        return e.detach(), g
