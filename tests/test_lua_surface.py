"""Static checks of the LuaJIT FFI file (no Lua toolchain exists where the tests run).

The file is what a Torch7 installation loads in place of
fbcunn/SpatialConvolutionFBFFT.lua.  Checked here: its blocks balance, the C prototypes
in its ffi.cdef agree with include/fbfftconv.h argument by argument, and the methods and
fields the reference's callers use are present (fbcunn/SpatialConvolutionFBFFT.lua:102,
:189, :269; fbcunn/SpatialConvolutionFFT.lua:162-163, :259-268).
"""
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
LUA = os.path.join(ROOT, "fbcunn_b200", "lua", "SpatialConvolutionFBFFT.lua")
HEADER = os.path.join(ROOT, "include", "fbfftconv.h")


def _lua_text():
    with open(LUA) as f:
        return f.read()


def _strip_lua(text, keep_cdef=False):
    """Removes comments and string literals (the ffi.cdef block is a long string)."""
    out = re.sub(r"--\[\[.*?\]\]", "", text, flags=re.S)
    if not keep_cdef:
        out = re.sub(r"\[\[.*?\]\]", "''", out, flags=re.S)
    out = re.sub(r"--[^\n]*", "", out)
    out = re.sub(r"'(?:\\.|[^'\\\n])*'", "''", out)
    out = re.sub(r'"(?:\\.|[^"\\\n])*"', '""', out)
    return out


def test_blocks_balance():
    words = re.findall(r"[A-Za-z_][A-Za-z_0-9]*", _strip_lua(_lua_text()))
    opens = sum(words.count(w) for w in ("function", "if", "do"))
    assert words.count("repeat") == words.count("until")
    assert opens == words.count("end"), (opens, words.count("end"))
    code = _strip_lua(_lua_text())
    for a, b in ("()", "{}", "[]"):
        assert code.count(a) == code.count(b), (a, code.count(a), code.count(b))


def _prototypes(text):
    """name -> list of parameter types with the parameter names dropped."""
    protos = {}
    for ret, name, args in re.findall(
            r"\b(int|size_t|const char\s*\*|fbfftconv_handle\s*\*)\s+(fbfftconv_[a-z0-9_]+)\s*\(([^)]*)\)\s*;", text):
        types = []
        for a in [x.strip() for x in args.split(",")]:
            if a in ("void", ""):
                continue
            a = a.replace("fbfftconv_stream", "void*")
            a = re.sub(r"\s*\*\s*", "* ", a).strip()
            parts = a.split()
            if len(parts) > 1 and re.fullmatch(r"[A-Za-z_][A-Za-z_0-9]*", parts[-1]) and parts[-1] not in ("int", "float"):
                parts = parts[:-1]  # the parameter's name
            types.append(" ".join(parts))
        protos[name] = (re.sub(r"\s+", " ", ret), types)
    return protos


def test_cdef_matches_the_header():
    with open(HEADER) as f:
        header = re.sub(r"/\*.*?\*/", "", f.read(), flags=re.S)
    declared = _prototypes(header)
    cdef = re.search(r"ffi\.cdef\[\[(.*?)\]\]", _lua_text(), flags=re.S).group(1)
    bound = _prototypes(cdef)
    assert len(bound) >= 8
    for name, proto in bound.items():
        assert name in declared, f"{name} is bound by the Lua file but not declared in the header"
        assert proto == declared[name], (name, proto, declared[name])
    # the struct the Lua side fills must have the header's fields in the header's order
    def fields(text):
        body = re.search(r"typedef struct fbfftconv_desc\s*\{(.*?)\}", text, flags=re.S).group(1)
        names = []
        for decl in body.split(";"):
            decl = decl.strip()
            if decl:
                names += [n.strip() for n in re.sub(r"^(u?int32_t)\s+", "", decl).split(",")]
        return names
    assert fields(cdef) == fields(header)


def test_surface_of_the_reference_module():
    code = _strip_lua(_lua_text())
    for method in ("__init", "reset", "updateOutput", "updateGradInput", "accGradParameters", "backward",
                   "updateOutputFFTImpl", "updateGradInputFFTImpl", "accGradParametersFFTImpl",
                   "setReuseInputs", "setReuseOutputs", "setReuseWeights", "cleanupBuffers"):
        assert re.search(r"function SpatialConvolutionFBFFT:%s\(" % method, code), method
    for field in ("printDebugLevel", "cudnnDebug", "success", "autotuningPass", "reportErrors", "timeSteps",
                  "nInputPlane", "nOutputPlane", "kW", "kH", "dW", "dH", "padLeft", "padUp", "padRight", "padDown",
                  "memoryReusePolicy", "numCudaStreams", "weight", "bias", "gradWeight", "gradBias"):
        assert re.search(r"self\.%s\b" % field, code), field
    text = _lua_text()
    assert "torch.class('nn.SpatialConvolutionFBFFT'" in text
    assert "torch.class('nn.SpatialConvolutionFBFFTGemm', 'nn.SpatialConvolutionFBFFT')" in text
    # the tiled class of the reference (fbcunn/SpatialConvolutionFFTTiled.lua:265-267) over the tiled entry points
    assert "torch.class('nn.SpatialConvolutionFFTTiled', 'nn.SpatialConvolutionFBFFT')" in text
    for method in ("__init", "updateOutputFFTImpl", "updateGradInputFFTImpl", "accGradParametersFFTImpl",
                   "cleanupBuffers"):
        assert re.search(r"function SpatialConvolutionFFTTiled:%s\(" % method, code), method
    for call in ("fbfftconv_tiled_create", "fbfftconv_tiled_update_output", "fbfftconv_tiled_update_grad_input",
                 "fbfftconv_tiled_acc_grad_parameters"):
        assert "C." + call in code, call
    # skipBias must really switch the bias off: `x and nil or y` never does
    assert not re.search(r"and nil\)? or", code)
    assert code.count("metaData.skipBias") >= 2
