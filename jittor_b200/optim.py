"""The optimiser step either side of the path: gradients of the lazy graph, their data-parallel synchronisation and the
parameter update, with the reference's semantics (python/jittor/optim.py:18-345,389-438):

    backward(loss)   grads = jt.grad(loss, params); under data parallelism every gradient becomes its mean over the
                     ranks (optim.py:189-198) and every `param_sync_iter` steps the parameters are re-broadcast from
                     rank 0 (optim.py:199-202); gradients accumulate until zero_grad (optim.py:205-219).
    SGD.step         dp = p*weight_decay + g; v = momentum*v + dp*(1-dampening); p -= lr * (v | dp + momentum*v).
    Adam.step        m, v moments and the bias-corrected step of optim.py:420-437.

What differs is the exchange: the reference issues one all-reduce per gradient; here all gradients of a dtype travel
packed in a few flat buckets (`dist.all_reduce_buckets`), each reduced by the NVLink peer kernel (or NCCL when it does
not apply), and the division by the world size is the first op of the update chain the CUDA element-wise kernels run."""
import math

from . import dist
from . import var as V
from .grad import grad as _grad


class Optimizer:
    def __init__(self, params, lr, param_sync_iter=10000):
        params = list(params)
        assert len(params) > 0, "Length of parameters should not be zero"
        if not isinstance(params[0], dict):
            params = [{"params": params}]
        self.param_groups = []
        for pg in params:
            assert isinstance(pg, dict)
            pg["params"] = list(pg["params"])
            self.param_groups.append(pg)
        self.lr = lr
        self.param_sync_iter = param_sync_iter
        self.n_step = 0
        self._zero_grad = True

    def add_param_group(self, group):
        group["params"] = list(group["params"])
        self.param_groups.append(group)

    def zero_grad(self):
        self._zero_grad = True

    def backward(self, loss, retain_graph=False):
        params = [p for pg in self.param_groups for p in pg["params"]]
        with_grad = [p for p in params if not p.is_stop_grad()]
        for p in with_grad:
            p.sync()
        grads = _grad(loss, with_grad)
        if dist.in_mpi():
            for g in grads:
                g.sync()
            world = dist.world_size()
            summed = dist.all_reduce_buckets([g.wait()._data for g in grads])
            grads = [V.Var(g.shape, g.dtype, data=t) / world for g, t in zip(grads, summed)]
            if self.n_step % self.param_sync_iter == 0:
                for p in params:
                    p.assign(dist.mpi_broadcast(p))
        self.n_step += 1
        pid = 0
        for pg in self.param_groups:
            if "grads" not in pg:
                pg["grads"] = [V.zeros(list(p.shape), p.dtype) for p in pg["params"]]
            for i, p in enumerate(pg["params"]):
                if p.is_stop_grad():
                    continue
                g = grads[pid]
                pid += 1
                if not self._zero_grad:
                    g = g + pg["grads"][i]
                pg["grads"][i] = g.sync()
        self._zero_grad = False

    def pre_step(self, loss, retain_graph=False):
        if loss is not None:
            self.backward(loss, retain_graph)

    def post_step(self):
        self.zero_grad()

    def step(self, loss=None, retain_graph=False):
        self.pre_step(loss, retain_graph)
        for pg in self.param_groups:
            lr = pg.get("lr", self.lr)
            for p, g in zip(pg["params"], pg["grads"]):
                if p.is_stop_grad():
                    continue
                p.update(p - g * lr)
        self.post_step()

    def find_grad(self, v):
        for pg in self.param_groups:
            for p, g in zip(pg["params"], pg.get("grads", ())):
                if p is v:
                    return g
        raise RuntimeError("This variable is not managed by this optimizer")


class SGD(Optimizer):
    """python/jittor/optim.py:298-345."""

    def __init__(self, params, lr, momentum=0, weight_decay=0, dampening=0, nesterov=False):
        super().__init__(params, lr)
        self.momentum, self.weight_decay, self.dampening, self.nesterov = momentum, weight_decay, dampening, nesterov
        for pg in self.param_groups:
            pg["values"] = [V.zeros(list(p.shape), p.dtype) for p in pg["params"]]

    def add_param_group(self, group):
        group["values"] = [V.zeros(list(p.shape), p.dtype) for p in group["params"]]
        super().add_param_group(group)

    def step(self, loss=None, retain_graph=False):
        self.pre_step(loss, retain_graph)
        for pg in self.param_groups:
            lr = pg.get("lr", self.lr)
            momentum = pg.get("momentum", self.momentum)
            weight_decay = pg.get("weight_decay", self.weight_decay)
            dampening = pg.get("dampening", self.dampening)
            nesterov = pg.get("nesterov", self.nesterov)
            for i, (p, g) in enumerate(zip(pg["params"], pg["grads"])):
                if p.is_stop_grad():
                    continue
                v = pg["values"][i]
                dp = p * weight_decay + g
                v.update(v * momentum + dp * (1 - dampening))
                if nesterov:
                    p.update(p - (dp + v * momentum) * lr)
                else:
                    p.update(p - v * lr)
        self.post_step()


class Adam(Optimizer):
    """python/jittor/optim.py:389-438."""

    def __init__(self, params, lr, eps=1e-8, betas=(0.9, 0.999), weight_decay=0):
        super().__init__(params, lr)
        self.eps, self.betas, self.weight_decay = eps, betas, weight_decay
        for pg in self.param_groups:
            pg["values"] = [V.zeros(list(p.shape), p.dtype) for p in pg["params"]]
            pg["m"] = [V.zeros(list(p.shape), p.dtype) for p in pg["params"]]

    def step(self, loss=None, retain_graph=False):
        self.pre_step(loss, retain_graph)
        n = float(self.n_step)
        for pg in self.param_groups:
            lr = pg.get("lr", self.lr)
            eps = pg.get("eps", self.eps)
            weight_decay = pg.get("weight_decay", self.weight_decay)
            b0, b1 = pg.get("betas", self.betas)
            for i, (p, g) in enumerate(zip(pg["params"], pg["grads"])):
                if p.is_stop_grad():
                    continue
                v, m = pg["values"][i], pg["m"][i]
                g = p * weight_decay + g
                m.update(m * b0 + g * (1 - b0))
                v.update(v * b1 + g * g * (1 - b1))
                step_size = lr * math.sqrt(1 - b1 ** n) / (1 - b0 ** n)
                p.update(p - m * step_size / (V.unary(v, "sqrt") + eps))
        self.post_step()


class RMSprop(Optimizer):
    """python/jittor/optim.py:347-387."""

    def __init__(self, params, lr=1e-2, eps=1e-8, alpha=0.99):
        super().__init__(params, lr)
        self.eps, self.alpha = eps, alpha
        for pg in self.param_groups:
            pg["values"] = [V.zeros(list(p.shape), p.dtype) for p in pg["params"]]

    def add_param_group(self, group):
        group["values"] = [V.zeros(list(p.shape), p.dtype) for p in group["params"]]
        super().add_param_group(group)

    def step(self, loss=None, retain_graph=False):
        self.pre_step(loss, retain_graph)
        for pg in self.param_groups:
            lr, eps, alpha = pg.get("lr", self.lr), pg.get("eps", self.eps), pg.get("alpha", self.alpha)
            for i, (p, g) in enumerate(zip(pg["params"], pg["grads"])):
                if p.is_stop_grad():
                    continue
                v = pg["values"][i]
                v.update(v * alpha + g * g * (1 - alpha))
                p.update(p - g * lr / (V.unary(v, "sqrt") + eps))
        self.post_step()


class AdamW(Adam):
    """python/jittor/optim.py:440-491: decoupled weight decay, bias corrections applied to the denominator."""

    def step(self, loss=None, retain_graph=False):
        self.pre_step(loss, retain_graph)
        n = float(self.n_step)
        for pg in self.param_groups:
            lr = pg.get("lr", self.lr)
            eps = pg.get("eps", self.eps)
            weight_decay = pg.get("weight_decay", self.weight_decay)
            b0, b1 = pg.get("betas", self.betas)
            for i, (p, g) in enumerate(zip(pg["params"], pg["grads"])):
                if p.is_stop_grad():
                    continue
                v, m = pg["values"][i], pg["m"][i]
                p.update(p * (1 - lr * weight_decay))
                m.update(m * b0 + g * (1 - b0))
                v.update(v * b1 + g * g * (1 - b1))
                denom = V.unary(v, "sqrt") / math.sqrt(1 - b1 ** n) + eps
                p.update(p - m * (lr / (1 - b0 ** n)) / denom)
        self.post_step()
