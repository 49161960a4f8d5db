"""The optimiser step either side of the path: gradients of the lazy graph, their data-parallel synchronisation and the
parameter update, with the reference's semantics (python/jittor/optim.py:18-345,347-491):

    backward(loss)   grads = jt.grad(loss, params); under data parallelism every gradient becomes its mean over the
                     ranks (optim.py:189-198) and every `param_sync_iter` steps the parameters are re-broadcast from
                     rank 0 (optim.py:199-202); gradients accumulate until zero_grad (optim.py:205-219).
    SGD              dp = p*weight_decay + g; v = momentum*v + dp*(1-dampening); p -= lr * (v | dp + momentum*v).
    Adam / AdamW     first and second moments with the bias corrections of optim.py:420-437 / :471-491.
    RMSprop          v = alpha*v + (1-alpha)*g*g; p -= lr*g / (sqrt(v) + eps)  (optim.py:376-387).

What differs is the exchange: the reference issues one all-reduce per gradient; here all gradients of a dtype travel
packed in a few flat buckets (`dist.all_reduce_buckets`), each reduced by the NVLink peer kernel (or NCCL when it does
not apply), and the division by the world size is the first op of the update chain the CUDA element-wise kernels run.

Layout of this module: an optimiser class names its per-parameter state slots (`STATE`) and its hyper-parameters
(`HYPER`, each overridable per parameter group as in the reference) and implements one rule, `_update`; the walk over
groups and parameters, gradient bookkeeping and synchronisation live in the base class."""
import math

from . import dist
from . import var as V
from .grad import grad as _grad


def _zeros_like(p):
    return V.zeros(list(p.shape), p.dtype)


class Optimizer:
    STATE = ()          # names of per-parameter state lists kept in every parameter group
    HYPER = ()          # names of hyper-parameters looked up in the group first, then on the optimiser

    def __init__(self, params, lr, param_sync_iter=10000):
        groups = list(params)
        assert len(groups) > 0, "Length of parameters should not be zero"
        if not isinstance(groups[0], dict):
            groups = [{"params": groups}]
        self.lr, self.param_sync_iter, self.n_step = lr, param_sync_iter, 0
        self.param_groups = []
        self._zero_grad = True
        for group in groups:
            assert isinstance(group, dict)
            self.add_param_group(group)

    def add_param_group(self, group):
        group["params"] = list(group["params"])
        for slot in self.STATE:
            group[slot] = [_zeros_like(p) for p in group["params"]]
        self.param_groups.append(group)

    # ---- gradients --------------------------------------------------------------------------------------------
    def zero_grad(self):
        self._zero_grad = True

    def _all_params(self):
        return [p for group in self.param_groups for p in group["params"]]

    def backward(self, loss, retain_graph=False):
        everything = self._all_params()
        trainable = [p for p in everything if not p.is_stop_grad()]
        for p in trainable:
            p.sync()
        grads = _grad(loss, trainable)
        if dist.in_mpi():
            grads = self._synchronise(grads, everything)
        self.n_step += 1
        fresh = iter(grads)
        for group in self.param_groups:
            held = group.setdefault("grads", [_zeros_like(p) for p in group["params"]])
            for i, p in enumerate(group["params"]):
                if p.is_stop_grad():
                    continue
                g = next(fresh)
                held[i] = (g if self._zero_grad else g + held[i]).sync()
        self._zero_grad = False

    def _synchronise(self, grads, everything):
        """Mean of every gradient over the ranks (bucketed), and the periodic re-broadcast of the parameters."""
        for g in grads:
            g.sync()
        world = dist.world_size()
        summed = dist.all_reduce_buckets([g.wait()._data for g in grads])
        grads = [V.Var(g.shape, g.dtype, data=t) / world for g, t in zip(grads, summed)]
        if self.n_step % self.param_sync_iter == 0:
            for p in everything:
                p.assign(dist.mpi_broadcast(p))
        return grads

    def find_grad(self, v):
        for group in self.param_groups:
            for p, g in zip(group["params"], group.get("grads", ())):
                if p is v:
                    return g
        raise RuntimeError("This variable is not managed by this optimizer")

    # ---- the step ---------------------------------------------------------------------------------------------
    def pre_step(self, loss, retain_graph=False):
        if loss is not None:
            self.backward(loss, retain_graph)

    def post_step(self):
        self.zero_grad()

    def step(self, loss=None, retain_graph=False):
        self.pre_step(loss, retain_graph)
        for group in self.param_groups:
            hyper = {"lr": group.get("lr", self.lr)}
            for name in self.HYPER:
                hyper[name] = group.get(name, getattr(self, name))
            for i, p in enumerate(group["params"]):
                if not p.is_stop_grad():
                    self._update(p, group["grads"][i], {slot: group[slot][i] for slot in self.STATE}, hyper)
        self.post_step()

    def _update(self, p, g, state, h):
        """Plain gradient descent (optim.py:259-266)."""
        p.update(p - g * h["lr"])


class SGD(Optimizer):
    """python/jittor/optim.py:298-345."""
    STATE = ("values",)
    HYPER = ("momentum", "weight_decay", "dampening", "nesterov")

    def __init__(self, params, lr, momentum=0, weight_decay=0, dampening=0, nesterov=False):
        self.momentum, self.weight_decay, self.dampening, self.nesterov = momentum, weight_decay, dampening, nesterov
        super().__init__(params, lr)

    def _update(self, p, g, state, h):
        v = state["values"]
        dp = p * h["weight_decay"] + g
        v.update(v * h["momentum"] + dp * (1 - h["dampening"]))
        p.update(p - ((dp + v * h["momentum"]) if h["nesterov"] else v) * h["lr"])


class RMSprop(Optimizer):
    """python/jittor/optim.py:347-387."""
    STATE = ("values",)
    HYPER = ("eps", "alpha")

    def __init__(self, params, lr=1e-2, eps=1e-8, alpha=0.99):
        self.eps, self.alpha = eps, alpha
        super().__init__(params, lr)

    def _update(self, p, g, state, h):
        v = state["values"]
        v.update(v * h["alpha"] + g * g * (1 - h["alpha"]))
        p.update(p - g * h["lr"] / (V.unary(v, "sqrt") + h["eps"]))


class Adam(Optimizer):
    """python/jittor/optim.py:389-438."""
    STATE = ("values", "m")
    HYPER = ("eps", "betas", "weight_decay")

    def __init__(self, params, lr, eps=1e-8, betas=(0.9, 0.999), weight_decay=0):
        self.eps, self.betas, self.weight_decay = eps, betas, weight_decay
        super().__init__(params, lr)

    def _moments(self, g, state, h):
        b0, b1 = h["betas"]
        m, v = state["m"], state["values"]
        m.update(m * b0 + g * (1 - b0))
        v.update(v * b1 + g * g * (1 - b1))
        n = float(self.n_step)
        return m, v, 1 - b0 ** n, 1 - b1 ** n

    def _update(self, p, g, state, h):
        m, v, c0, c1 = self._moments(p * h["weight_decay"] + g, state, h)
        p.update(p - m * (h["lr"] * math.sqrt(c1) / c0) / (V.unary(v, "sqrt") + h["eps"]))


class AdamW(Adam):
    """python/jittor/optim.py:440-491: decoupled weight decay, bias corrections applied to the denominator."""

    def _update(self, p, g, state, h):
        p.update(p * (1 - h["lr"] * h["weight_decay"]))
        m, v, c0, c1 = self._moments(g, state, h)
        p.update(p - m * (h["lr"] / c0) / (V.unary(v, "sqrt") / math.sqrt(c1) + h["eps"]))
