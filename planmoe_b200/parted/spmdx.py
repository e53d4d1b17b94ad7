"""parted: describe a computation as a graph of einsum-like nodes, search a sharding plan, and
emit a runnable SPMD PyTorch program.

API parity with ``PlanMoE/parted/spmdx.py:17-597``: ``init(backend)``, ``Tensor``, ``Id``,
``Custom`` (with ``autotune`` / ``compile`` / ``get_data_parallel_config``), ``Program``
(``save`` / ``execute``) and the version-0.1 JSON ``Config`` ``{v, t, b, kwargs}``; environment
switches ``STRICT_FMT``, ``PTYPE`` (dp | zero), ``CONFIG`` (manual states), ``DEVICE``, ``MODE``,
``CONFIG_STORE_PATH``.

A node's tensor format is ``"out[+] = in0, in1"`` where each letter is an axis, ``(ab)`` fuses two
axes into one dim, and a trailing ``+`` on the left marks a sum over the axes that do not appear in
the output.  ``fw_ops`` is the PyTorch expression that computes the node; inputs are referenced by
interpolating the input objects (``f"torch.matmul({x}, {w})"``).
"""

import importlib
import inspect
import json
import logging
import os
import re
import tempfile

from . import patterns  # noqa: F401  (registers the primitives)
from . import solver

session = None


class _Session:
    def __init__(self, backend_name):
        self.backend = importlib.import_module('planmoe_b200.parted.backend.%s.config' % backend_name)
        self.is_strict_fmt = int(os.environ.get('STRICT_FMT', 0)) > 0
        self.ptype = os.environ.get('PTYPE', '')
        self.custom_dict = {}
        self.counters = {}
        manual = os.environ.get('CONFIG', '')
        manual = json.loads(manual) if manual else {}
        self.manual_config = {k: (v if isinstance(v, int) else v[0]) for k, v in manual.items()}


def init(backend_name, reset=False):
    """Create the (single) session for ``backend_name`` ('torch')."""
    global session
    if session is not None and not reset:
        raise Exception('Function `init()` can be only invoked once.')
    if not re.match(r'^[a-zA-Z0-9]+$', backend_name):
        raise Exception('Only letters and digits are allowed for backend_name, get: %s' % backend_name)
    session = _Session(backend_name)
    try:
        return importlib.import_module('planmoe_b200.parted.backend.%s' % backend_name)
    except ImportError:
        return None


def new_dependency(header_content, depends=()):
    depends = list(depends) if isinstance(depends, (list, tuple)) else [depends]
    return {'data': header_content.strip() + '\n', 'depends': depends}


def product(values):
    out = 1
    for v in values:
        out *= int(v)
    return out


class Mapper2D:
    """One side of a tensor format: ``id2ax[i]`` is the axis letter of dim i (or a list of letters
    for a fused dim); ``ax2id[letter]`` is the dim index (or ``(dim, position)`` inside a fused dim)."""

    def __init__(self, text):
        self.id2ax = []
        fused = None
        for ch in text:
            if ch.isspace():
                continue
            if ch == '(':
                fused = []
            elif ch == ')':
                self.id2ax.append(fused if len(fused) > 1 else fused[0])
                fused = None
            elif fused is not None:
                fused.append(ch)
            else:
                self.id2ax.append(ch)
        self.ax2id = {}
        for i, ax in enumerate(self.id2ax):
            if isinstance(ax, str):
                if ax != '*':
                    self.ax2id[ax] = i
            else:
                for j, a in enumerate(ax):
                    self.ax2id[a] = (i, j)


class Parser:
    def __init__(self, ir):
        left, rights = ir.split('=')
        left = left.rstrip()
        self.reduce_type = ''
        if left and left[-1] in '+<>[]':
            left, self.reduce_type = left[:-1], left[-1]
        self.left = Mapper2D(left)
        self.rights = [Mapper2D(r) for r in rights.split(',')]
        self.num_inputs = len(self.rights)

    def get_reduce_axes(self):
        axes = set()
        for r in self.rights:
            for ax in r.ax2id:
                if ax not in self.left.ax2id:
                    axes.add(ax)
        return axes

    def emit_dims_by_name(self, ax):
        """For an axis: the dim of every input that carries it (-1 when absent), and how many do."""
        if ax == '*':
            raise NotImplementedError()
        lead = ax if isinstance(ax, str) else ax[0]
        dims, parted = {}, 0
        for i, r in enumerate(self.rights):
            where = r.ax2id.get(lead)
            if where is None:
                dims[i] = -1
                continue
            if isinstance(where, int):
                dims[i] = where
            elif where[1] == 0:
                dims[i] = where[0]
            else:
                raise NotImplementedError()     # sharding a non-leading member of a fused dim
            parted += 1
        return dims, parted

    def emit_dims_by_id(self, output_dim):
        if output_dim == -1:
            return {i: -1 for i in range(self.num_inputs)}, 0
        if output_dim < 0 or self.left.id2ax[output_dim] == '*':
            raise NotImplementedError()
        return self.emit_dims_by_name(self.left.id2ax[output_dim])


class Program:
    def __init__(self, code, kwargs):
        self.code, self.kwargs = code, kwargs

    def save(self, path):
        with open(path, 'w') as fp:
            fp.write(self.code)

    def execute(self, save_file_path=None):
        """Run the program on ``total_nodes`` ranks; returns the JSON record the executor wrote
        (``{'name', 'step_time'}``) or ``{}`` on failure."""
        temp = save_file_path is None
        if temp:
            fd, save_file_path = tempfile.mkstemp(suffix='.py')
            os.close(fd)
        self.save(save_file_path)
        fd, log_file = tempfile.mkstemp(suffix='.json')
        os.close(fd)
        os.unlink(log_file)
        os.environ['CONFIG_STORE_PATH'] = log_file
        cmd = session.backend.get_execute_cmd(self.kwargs['spmd_nodes'], self.kwargs['total_nodes'],
                                              self.kwargs['device_type'], save_file_path)
        result = {}
        try:
            logging.info('Executing: %s', cmd)
            if os.system(cmd) == 0 and os.path.exists(log_file):
                with open(log_file) as fp:
                    result = json.loads(fp.read().strip())
        except Exception as ex:
            logging.warning('program execution failed: %s', ex)
        finally:
            for f in ([save_file_path] if temp else []) + [log_file]:
                try:
                    os.unlink(f)
                except OSError:
                    pass
        return result


class Custom:
    def __init__(self, data, fw_ops=None, inputs=None, op_name=None, shape_fn=None, flops=None, depends=()):
        assert session is not None, "call spmdx.init('torch') first"
        self.op_type = op_name or inspect.currentframe().f_back.f_code.co_name
        if not re.match(r'^[a-zA-Z0-9]+$', self.op_type):
            self.op_type = 'Custom'
        assert self.op_type[0].isupper(), \
            'The leading charactor of the operator name must be uppercase letter (received: "%s").' % self.op_type
        n = session.counters.get(self.op_type, 0)
        session.counters[self.op_type] = n + 1
        self.name = '%s%s%d' % (self.op_type[0].lower(), self.op_type[1:], n)
        self.depends = list(depends) if isinstance(depends, (list, tuple)) else [depends]
        self.fw_ops = fw_ops.replace('@@', '') if fw_ops is not None else None
        self.outputs = []
        self.data = data

        if isinstance(data, dict):
            self.op_type = 'param' if data['is_param'] else 'data'
            if data['is_param']:
                self.name += '_'
            self.inputs = []
            self.shape, self.dtype = list(data['shape']), data['dtype']
            self.flops = flops or 0
        else:
            if inputs is None:
                assert fw_ops is not None, 'At least one property in "fw_ops" and inputs should be specified.'
                names = []
                for piece in fw_ops.split('@@')[1::2]:
                    if piece not in names:
                        names.append(piece)
                inputs = [session.custom_dict[x] for x in names]
            self.inputs = list(inputs)
            self.op_type = 'compute'
            self.parser = Parser(data)
            if shape_fn is not None:
                self.shape, self.dtype = shape_fn(self.inputs)
            else:
                size = {}
                for i, r in enumerate(self.parser.rights):
                    for ax, where in r.ax2id.items():
                        if isinstance(where, int):
                            size[ax] = self.inputs[i].shape[where]
                try:
                    self.shape = [size[a] if isinstance(a, str) else product(size[b] for b in a)
                                  for a in self.parser.left.id2ax]
                except KeyError:
                    raise Exception('Cannot auto-infershape for op %s due to unknown dimension size by tensor '
                                    'format: %s' % (self.name, self.data))
                self.dtype = self.inputs[0].dtype
            if flops is None:
                self.flops = product(self.shape)
                if self.parser.reduce_type:
                    size = {}
                    for i, r in enumerate(self.parser.rights):
                        for ax, where in r.ax2id.items():
                            if isinstance(where, int):
                                size[ax] = self.inputs[i].shape[where]
                    self.flops *= product(size.get(a, 1) for a in self.parser.get_reduce_axes())
                    self.flops *= 2
            else:
                self.flops = flops
        assert self.name not in session.custom_dict, "Node with name `%s` has already existed." % self.name
        session.custom_dict[self.name] = self

    def __str__(self):
        return '@@%s@@' % self.name

    def numel(self):
        return int(product(self.shape))

    # -- graph walks ---------------------------------------------------------------------------
    def _topo(self):
        order, seen = [], set()

        def visit(n):
            if id(n) in seen:
                return
            seen.add(id(n))
            for i in n.inputs:
                visit(i)
            order.append(n)
        visit(self)
        return order

    def update_config(self, parent, **kwargs):
        for n in self._topo():
            n.outputs = []
        for n in self._topo():
            for i in n.inputs:
                if n not in i.outputs:
                    i.outputs.append(n)
            if kwargs['spmd_nodes'] == 1:
                n.config = -1
            elif session.ptype == 'dp':
                n.config = -1 if n.op_type == 'param' else 0
            elif session.ptype == 'zero':
                n.config = -2 if n.op_type == 'param' else 0
            elif n.name in session.manual_config:
                n.config = session.manual_config[n.name]

    def serialize(self, **kwargs):
        self.update_config(None, **kwargs)
        order = self._topo()
        input_nodes = [n for n in order if isinstance(n.data, dict)]
        compute_nodes = [n for n in order if not isinstance(n.data, dict)]
        config = {n.name: n.config for n in order if hasattr(n, 'config')}
        multi = set(i for n in compute_nodes for i in n.inputs if len(i.outputs) > 1)
        return [(compute_nodes, multi)], compute_nodes, input_nodes, config

    def get_data_parallel_config(self, **kwargs):
        cfg = {n.name: ([-1, ''] if n.op_type == 'param' else [0, 'BAR:0']) for n in self._topo()}
        return Config.create(cfg, environ_config(kwargs))

    # -- plan search / code generation ---------------------------------------------------------------
    def autotune(self, config_file=None, **kwargs):
        cached = Config.load_from_file(config_file)
        if cached:
            return cached
        kwargs, results = optimize(self, **kwargs)
        valid = [sol for _, sol in results if sol is not None]
        if not valid:
            raise Exception('No valid configuration found!')
        best_time, best = min(valid, key=lambda s: s[0])
        cfg = Config.create(best, {k: v for k, v in kwargs.items()}, best_time)
        if config_file is not None:
            cfg.save(config_file)
        return cfg

    def compile(self, config, **kwargs):
        if not isinstance(config, dict):
            assert config.config['v'] == Config.VERSION
            merged = dict(config.config['kwargs'])
            merged.update(kwargs)
            kwargs, config = merged, config.config['b']
        kwargs = environ_config(kwargs)
        spmd = kwargs['spmd_nodes']
        _, compute_nodes, input_nodes, fixed = self.serialize(**kwargs)
        for n in compute_nodes + input_nodes:
            state = config[n.name][0]
            if fixed.get(n.name, state) != state:
                raise Exception('Unstatisfied sharding state requirements on node `%s`' % n.name)
            if state >= 0 and n.shape[state] % spmd != 0:
                raise Exception('Unstatisfied slicing chunks `%d // %d` on node `%s`' % (n.shape[state], spmd, n.name))

        input_list, param_list = [], []
        for n in input_nodes:
            code = session.backend.get_input_definition(n.name, n.shape, config[n.name][0], n.dtype,
                                                        is_param=(n.op_type == 'param'))
            (param_list if n.op_type == 'param' else input_list).append((n.name, code))

        lines, temp = [], 0
        for n in compute_nodes:
            out_state, key = config[n.name]
            rank = None
            if ':' in key:
                key, rank = key.split(':')
                rank = int(rank)
            found = list(solver.spmd_primitives_dict[key](session, n, out_state, spmd, rank))
            assert len(found) == 1, "pattern `%s` on node `%s` at state %s: %d solutions" % (key, n.name, out_state, len(found))
            _, want, conn = found[0]
            expr = n.fw_ops
            for idx, inp in enumerate(n.inputs):
                cur = inp.name
                have, need = config[inp.name][0], want[idx]
                extra = {'output_shape': inp.shape, 'is_param': inp.op_type == 'param'}
                if have != need:
                    if have == -2 and need >= 0:
                        cur = session.backend.link(cur, -2, -1, **extra)
                        cur = session.backend.link(cur, -1, need, **extra)
                    else:
                        cur = session.backend.link(cur, have, need, **extra)
                if conn.get(idx):
                    cur = conn[idx].replace('$', cur)
                if cur != inp.name:
                    temp += 1
                    lines.append('_temp%d = %s' % (temp, cur))
                    expr = re.sub(r'\b%s\b' % re.escape(inp.name), '_temp%d' % temp, expr)
            lines.append('%s = %s' % (n.name, expr))
            if conn.get(''):
                lines.append('%s = %s' % (n.name, conn[''].replace('$', n.name)))

        headers, seen = [], set()

        def add_dep(dep):
            if id(dep) in seen:
                return
            seen.add(id(dep))
            for d in dep['depends']:
                add_dep(d)
            headers.append(dep['data'])
        for n in compute_nodes:
            for d in n.depends:
                add_dep(d)

        code = session.backend.generate_framework_code(
            kwargs['device_type'], spmd, kwargs['total_nodes'] // spmd, kwargs['run_mode'], self.name, headers,
            input_list, param_list, lines)
        return Program(code, kwargs)


def environ_config(kwargs):
    kwargs = dict(kwargs)
    kwargs.setdefault('total_nodes', 1)
    kwargs.setdefault('spmd_nodes', kwargs['total_nodes'])
    kwargs.setdefault('device_type', os.environ.get('DEVICE', 'cuda'))
    kwargs.setdefault('run_mode', os.environ.get('MODE', 'train'))
    assert kwargs['total_nodes'] % kwargs['spmd_nodes'] == 0, "`total_nodes` must be exactly divided by `spmd_nodes`."
    return kwargs


def optimize(node, **kwargs):
    kwargs = environ_config(kwargs)
    if session.is_strict_fmt:
        node = Id(node, op_name='Builtin')
        node.config = 0
    groups, compute_nodes, input_nodes, config = node.serialize(**kwargs)
    return kwargs, solver.solve_partition(session, groups, input_nodes=input_nodes, split_pref=config, kwargs=kwargs)


class Config:
    VERSION = '0.1'

    @staticmethod
    def load_from_file(filename):
        if filename is not None and os.path.exists(filename):
            return Config(filename)
        return None

    @staticmethod
    def create(config, environ, timecost=0):
        return Config({'v': Config.VERSION, 't': timecost, 'b': config, 'kwargs': environ})

    def __init__(self, config):
        if isinstance(config, str):
            with open(config) as fp:
                config = json.load(fp)
        if not isinstance(config, dict):
            raise Exception('Unsupported config value: %s' % (config,))
        if config.get('v') != Config.VERSION:
            raise Exception('Incompatible config version: expect %s, got %s' % (Config.VERSION, config.get('v')))
        self.config = config

    def __str__(self):
        return json.dumps(self.config)

    def save(self, filepath):
        with open(filepath, 'w') as fp:
            json.dump(self.config, fp)


def Id(x, op_name=None):
    axes = ''.join(chr(ord('a') + i) for i in range(len(x.shape)))
    return Custom('%s = %s' % (axes, axes), '%s' % x, op_name=op_name or 'Id')


def Tensor(shape, dtype, is_param=False):
    node = Custom({'shape': shape, 'dtype': dtype, 'is_param': is_param}, inputs=[], op_name='Tensor')
    if not is_param and session.is_strict_fmt:
        state = session.manual_config.pop(node.name, None)
        node.config = 0
        node = Id(node, op_name='Builtin')
        if state is not None:
            node.config = state
    return node
