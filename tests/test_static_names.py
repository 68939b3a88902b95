"""Static scan for names that are read but never bound: branches that only run on a GPU box
(kernel wrappers, multi-GPU paths of bench.py) are not executed by the CPU suite, so a typo or
a variable from another scope would only surface there."""
import ast
import builtins
import os

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def check(path):
    src=open(path).read(); tree=ast.parse(src)
    glob=set(dir(builtins))|{'__file__','__name__','__doc__'}
    for n in tree.body:
        for m in ast.walk(n) if not isinstance(n,(ast.FunctionDef,ast.ClassDef)) else [n]:
            if isinstance(m,ast.Name) and isinstance(m.ctx,ast.Store): glob.add(m.id)
            if isinstance(m,(ast.FunctionDef,ast.ClassDef)): glob.add(m.name)
            if isinstance(m,(ast.Import,ast.ImportFrom)):
                for a in m.names: glob.add((a.asname or a.name).split('.')[0])
    star=any(isinstance(n,ast.ImportFrom) and any(a.name=='*' for a in n.names) for n in ast.walk(tree))
    out=[]
    def scope_names(fn):
        local=set()
        a=fn.args
        for x in a.args+a.kwonlyargs+a.posonlyargs: local.add(x.arg)
        if a.vararg: local.add(a.vararg.arg)
        if a.kwarg: local.add(a.kwarg.arg)
        return local
    def visit(fn, outer):
        local=scope_names(fn)|set(outer)
        body=fn.body if isinstance(fn.body,list) else [fn.body]
        stack=list(body); inner=[]
        nodes=[]
        while stack:
            n=stack.pop()
            nodes.append(n)
            if isinstance(n,(ast.FunctionDef,ast.Lambda,ast.AsyncFunctionDef)):
                if isinstance(n,ast.FunctionDef): local.add(n.name)
                inner.append(n); 
                # defaults/decorators evaluated in outer scope
                continue
            if isinstance(n,ast.ClassDef):
                local.add(n.name)
            stack.extend(ast.iter_child_nodes(n))
        for n in nodes:
            if isinstance(n,ast.Name) and isinstance(n.ctx,(ast.Store,ast.Del)): local.add(n.id)
            if isinstance(n,(ast.Import,ast.ImportFrom)):
                for a in n.names: local.add((a.asname or a.name).split('.')[0])
            if isinstance(n,ast.ExceptHandler) and n.name: local.add(n.name)
            if isinstance(n,(ast.Global,ast.Nonlocal)): local|=set(n.names)
            if isinstance(n,ast.arg): local.add(n.arg)
            if isinstance(n,ast.MatchAs) and n.name: local.add(n.name)
        for n in nodes:
            if isinstance(n,ast.Name) and isinstance(n.ctx,ast.Load) and n.id not in local and n.id not in glob and not star:
                out.append((getattr(fn,'name','<lambda>'),n.lineno,n.id))
        for f in inner: visit(f, local)
    for n in ast.walk(tree):
        pass
    def top(nodes, outer):
        for n in nodes:
            if isinstance(n,(ast.FunctionDef,ast.AsyncFunctionDef)): visit(n, outer)
            elif isinstance(n,ast.ClassDef):
                cls_names={m.name for m in n.body if isinstance(m,(ast.FunctionDef,ast.ClassDef))}|{t.id for m in n.body for t in ast.walk(m) if isinstance(m,(ast.Assign,ast.AnnAssign)) and isinstance(t,ast.Name) and isinstance(t.ctx,ast.Store)}
                top(n.body, outer)
    top(tree.body,set())
    return out


def _files():
    roots = ["necklace_b200", "benchmarks", "examples", "baseline/shims", "bench.py",
             "__graft_entry__.py", "baseline/ref_gpt2_zero.py", "baseline/torch_gpt2.py",
             "baseline/torch_resnet.py"]
    for r in roots:
        p = os.path.join(ROOT, r)
        if p.endswith(".py"):
            if os.path.exists(p):
                yield p
            continue
        for d, _, fs in os.walk(p):
            for f in fs:
                if f.endswith(".py"):
                    yield os.path.join(d, f)


def test_no_unbound_names_in_package_bench_and_examples():
    bad = [(os.path.relpath(f, ROOT),) + r for f in _files() for r in check(f)]
    assert not bad, bad


def test_the_scan_sees_an_unbound_name(tmp_path):
    p = tmp_path / "m.py"
    p.write_text("class A:\n    def __init__(self, x):\n        self.x = x\n"
                 "        if which == 4:\n            pass\n")
    assert check(str(p)) == [("__init__", 4, "which")]
