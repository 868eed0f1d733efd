#!/usr/bin/env python3
"""Make the golden files of this folder with the reference's own C code.

popixoxipop-collab/beglin's model file (qwen_infer.c) needs Apple's Accelerate and ARM NEON and does
not compile whole on an x86 Linux host.  Its loaders and its frequency-scaling header do compile with
plain gcc, and so do the functions of the model's arithmetic when they are taken out of the file by
their lines: they call a dozen Accelerate routines, each a loop that a shim restates.  This script
compiles, into a scratch folder, hf_config.c + hf_config_verify.c, safetensors_load.c +
safetensors_quants.c + safetensors_verify.c, a six-line driver around rope_llama3_scale.h, and a model
driver (below), and runs them on model folders written by this framework's random-weights mode:

    config_<name>.txt        the fields the reference reads from config.json (hf_config_verify.c)
    checksums_<name>.txt     one weighted checksum per tensor (safetensors_verify.c:24-27)
    rope_scale_<name>.txt    the llama3 frequency ratios (rope_llama3_scale.h:18-28)
    model_<name>.txt         a tiny random model run token by token by the reference's own functions:
                             cosines and sines of some positions, the logits of some positions of a
                             seeded sequence, and greedy tokens that continue it

The model driver `#include`s these lines of qwen_infer.c, cut out at run time (nothing of them is kept
in this repository): the configuration struct (:64-69), rmsnorm, softmax_inplace and swiglu (:711-733),
rope_head, rope_apply and rope_precompute (:765-794), the cache's slot functions (:796-798), the loop over
heads of the plain attention branch (:1538-1543) and argmax_v (:2155).  Around them it has a shim of the
Accelerate calls they make (plain float loops) and a main that reads the weights and runs the layers in
the order of forward_token (:1435-1584) and final_logits (:1585-1599); that glue is written here.

tests/test_golden.py compares this framework's readers and the plain implementation with these files
(and, where the reference tree and gcc are present, with fresh runs of the same programs).

    python tests/golden/make_golden.py /path/to/reference
"""
import json
import os
import subprocess
import sys
import tempfile

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

ROPE_DRIVER = r'''
#include <stdio.h>
#include <stdlib.h>
#include "rope_llama3_scale.h"
int main(int argc, char **argv) {
    float theta = atof(argv[1]); int hd = atoi(argv[2]);
    float factor = atof(argv[3]), low = atof(argv[4]), high = atof(argv[5]), orig = atof(argv[6]);
    for (int i = 0; i < hd / 2; i++) printf("%d %.9g\n", i, rope_llama3_scale(theta, hd, factor, low, high, orig, i));
    return 0;
}
'''


# (first line, last line, text the first line must contain): the slices of qwen_infer.c the model driver includes
MODEL_SLICES = {
    "cfg": (64, 69, "typedef struct {"),
    "primitives": (711, 733, "static void rmsnorm("),
    "rope": (765, 794, "static void rope_head("),
    "cache": (796, 798, "static float *g_kcache, *g_vcache;"),
    "attention": (1538, 1543, "for(int h=0;h<g_cfg.nh;h++){ int kvh=h/g_cfg.group;"),
    "argmax": (2155, 2155, "static inline int argmax_v("),
}

MODEL_DRIVER = r'''
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <math.h>
/* ---- a shim of the Accelerate routines the slices call: the documented loops, in float ---- */
typedef unsigned long vDSP_Length;
static void vDSP_svesq(const float *a, long ia, float *c, vDSP_Length n) { float s = 0.0f; for (vDSP_Length i = 0; i < n; i++) s += a[i*ia]*a[i*ia]; *c = s; }
static void vDSP_maxv(const float *a, long ia, float *c, vDSP_Length n) { float m = -INFINITY; for (vDSP_Length i = 0; i < n; i++) if (a[i*ia] > m) m = a[i*ia]; *c = m; }
static void vDSP_maxvi(const float *a, long ia, float *c, vDSP_Length *ci, vDSP_Length n) { float m = -INFINITY; vDSP_Length at = 0; for (vDSP_Length i = 0; i < n; i++) if (a[i*ia] > m) { m = a[i*ia]; at = i*ia; } *c = m; *ci = at; }
static void vDSP_vsadd(const float *a, long ia, const float *b, float *c, long ic, vDSP_Length n) { for (vDSP_Length i = 0; i < n; i++) c[i*ic] = a[i*ia] + *b; }
static void vDSP_vsmul(const float *a, long ia, const float *b, float *c, long ic, vDSP_Length n) { for (vDSP_Length i = 0; i < n; i++) c[i*ic] = a[i*ia] * *b; }
static void vDSP_sve(const float *a, long ia, float *c, vDSP_Length n) { float s = 0.0f; for (vDSP_Length i = 0; i < n; i++) s += a[i*ia]; *c = s; }
static void vDSP_vneg(const float *a, long ia, float *c, long ic, vDSP_Length n) { for (vDSP_Length i = 0; i < n; i++) c[i*ic] = -a[i*ia]; }
static void vDSP_vdiv(const float *b, long ib, const float *a, long ia, float *c, long ic, vDSP_Length n) { for (vDSP_Length i = 0; i < n; i++) c[i*ic] = a[i*ia] / b[i*ib]; }   /* c = a / b: the divisor comes first */
static void vDSP_vmul(const float *a, long ia, const float *b, long ib, float *c, long ic, vDSP_Length n) { for (vDSP_Length i = 0; i < n; i++) c[i*ic] = a[i*ia] * b[i*ib]; }
static void vDSP_vadd(const float *a, long ia, const float *b, long ib, float *c, long ic, vDSP_Length n) { for (vDSP_Length i = 0; i < n; i++) c[i*ic] = a[i*ia] + b[i*ib]; }
static void vDSP_dotpr(const float *a, long ia, const float *b, long ib, float *c, vDSP_Length n) { float s = 0.0f; for (vDSP_Length i = 0; i < n; i++) s += a[i*ia]*b[i*ib]; *c = s; }
static void vDSP_vsma(const float *a, long ia, const float *b, const float *c, long ic, float *d, long id, vDSP_Length n) { for (vDSP_Length i = 0; i < n; i++) d[i*id] = a[i*ia] * *b + c[i*ic]; }
static void vvexpf(float *y, const float *x, const int *n) { for (int i = 0; i < *n; i++) y[i] = expf(x[i]); }
#define AHD 128
#define AGROUP 6
#include "slice_cfg.inc"
static int g_rope_norm = 0;
static float *g_rope_scale;
#include "rope_llama3_scale.h"
#include "slice_primitives.inc"
#include "slice_rope.inc"
#include "slice_cache.inc"
#include "slice_argmax.inc"
static float *q, *scores, *attn;
/* the plain attention branch of forward_token for one token at `pos` of layer l */
static void attention_plain(int l, int pos, float scale) {
#include "slice_attention.inc"
}
/* y = W x (+ b), W row-major [out, in]: what cblas_sgemv does for matvec_t's float branch (qwen_infer.c:688-691) */
static void matvec(const float *W, const float *b, const float *x, float *y, int out, int in) {
    for (int o = 0; o < out; o++) { float s = 0.0f; for (int i = 0; i < in; i++) s += W[(long)o*in+i]*x[i]; y[o] = s + (b ? b[o] : 0.0f); }
}
static float *take(float **p, long n) { float *r = *p; *p += n; return r; }
int main(int argc, char **argv) {
    /* argv: model.bin tokens.txt n_new ; model.bin: 12 int32 + 6 float32 of header, then float32 tensors in the order read below */
    FILE *f = fopen(argv[1], "rb"); if (!f) return 2;
    int hi[12]; float hf[6];
    if (fread(hi, 4, 12, f) != 12 || fread(hf, 4, 6, f) != 6) return 2;
    g_cfg.nl = hi[0]; g_cfg.d = hi[1]; g_cfg.nh = hi[2]; g_cfg.nkv = hi[3]; g_cfg.hd = hi[4]; g_cfg.im = hi[5]; g_cfg.vocab = hi[6];
    g_cfg.maxseq = hi[7]; g_cfg.qkv_bias = hi[8]; int tied = hi[9], scaled = hi[10];
    g_cfg.theta = hf[0]; g_cfg.eps = hf[1];
    g_cfg.kvd = g_cfg.nkv*g_cfg.hd; g_cfg.qd = g_cfg.nh*g_cfg.hd; g_cfg.group = g_cfg.nh/g_cfg.nkv;     /* qwen_infer.c:19478-19482 */
    long pos0 = ftell(f); fseek(f, 0, SEEK_END); long n_floats = (ftell(f) - pos0) / 4; fseek(f, pos0, SEEK_SET);
    float *all = malloc(n_floats*4); if (fread(all, 4, n_floats, f) != (size_t)n_floats) return 2; fclose(f);
    float *p = all;
    int d = g_cfg.d, qd = g_cfg.qd, kvd = g_cfg.kvd, im = g_cfg.im, V = g_cfg.vocab, NL = g_cfg.nl, hd = g_cfg.hd;
    float *embed = take(&p, (long)V*d);
    float **ln1 = malloc(NL*sizeof(float*)), **ln2 = malloc(NL*sizeof(float*)), **wq = malloc(NL*sizeof(float*)), **wk = malloc(NL*sizeof(float*)),
          **wv = malloc(NL*sizeof(float*)), **wo = malloc(NL*sizeof(float*)), **bq = malloc(NL*sizeof(float*)), **bk = malloc(NL*sizeof(float*)),
          **bv = malloc(NL*sizeof(float*)), **wg = malloc(NL*sizeof(float*)), **wu = malloc(NL*sizeof(float*)), **wd = malloc(NL*sizeof(float*));
    for (int l = 0; l < NL; l++) {
        ln1[l] = take(&p, d); wq[l] = take(&p, (long)qd*d); wk[l] = take(&p, (long)kvd*d); wv[l] = take(&p, (long)kvd*d);
        bq[l] = g_cfg.qkv_bias ? take(&p, qd) : NULL; bk[l] = g_cfg.qkv_bias ? take(&p, kvd) : NULL; bv[l] = g_cfg.qkv_bias ? take(&p, kvd) : NULL;
        wo[l] = take(&p, (long)d*qd); ln2[l] = take(&p, d); wg[l] = take(&p, (long)im*d); wu[l] = take(&p, (long)im*d); wd[l] = take(&p, (long)d*im);
    }
    float *final_norm = take(&p, d);
    float *head = tied ? embed : take(&p, (long)V*d);                /* the head is the table unless lm_head exists (qwen_infer.c:318-319) */
    if (p - all != n_floats) { fprintf(stderr, "model.bin: %ld floats left over\n", (long)(n_floats - (p - all))); return 2; }
    g_rope_scale = malloc(sizeof(float)*hd/2);
    for (int i = 0; i < hd/2; i++)                                    /* init_rope_scale, qwen_infer.c:757-764 */
        g_rope_scale[i] = scaled ? rope_llama3_scale(g_cfg.theta, hd, hf[2], hf[3], hf[4], hf[5], i) : 1.0f;
    int ids[4096], n_ids = 0, n_new = atoi(argv[3]);
    FILE *t = fopen(argv[2], "r"); while (n_ids < 4096 && fscanf(t, "%d", &ids[n_ids]) == 1) n_ids++; fclose(t);
    g_kcache = malloc(sizeof(float)*(long)NL*g_cfg.maxseq*kvd); g_vcache = malloc(sizeof(float)*(long)NL*g_cfg.maxseq*kvd);
    swiglu_tmp1 = malloc(sizeof(float)*im); swiglu_tmp2 = malloc(sizeof(float)*im);
    float *x = malloc(4*d), *h = malloc(4*d), *kv_k = malloc(4*kvd), *kv_v = malloc(4*kvd), *o = malloc(4*d), *gate = malloc(4*im),
          *up = malloc(4*im), *act = malloc(4*im), *m = malloc(4*d), *normed = malloc(4*d), *logits = malloc(4*V);
    q = malloc(4*qd); attn = malloc(4*qd); scores = malloc(4*g_cfg.maxseq);
    float *rc = malloc(4*hd/2), *rs = malloc(4*hd/2);
    /* cosines and sines of some positions (rope_precompute) */
    int far[5] = {0, 1, 77, 4000, 32767};
    for (int k = 0; k < 5; k++) { rope_precompute(far[k], rc, rs); printf("rope %d", far[k]); for (int i = 0; i < hd/2; i++) printf(" %.9g %.9g", rc[i], rs[i]); printf("\n"); }
    int total = n_ids + n_new - 1;
    for (int pos = 0; pos < total; pos++) {
        int id = ids[pos];
        memcpy(x, embed + (long)id*d, 4*d);                                           /* forward_token, qwen_infer.c:1438-1439 */
        rope_precompute(pos, rc, rs);
        for (int l = 0; l < NL; l++) {
            rmsnorm(x, ln1[l], h, d);
            matvec(wq[l], bq[l], h, q, qd, d); matvec(wk[l], bk[l], h, kv_k, kvd, d); matvec(wv[l], bv[l], h, kv_v, kvd, d);
            for (int hh = 0; hh < g_cfg.nh; hh++) rope_apply(q + hh*hd, rc, rs);
            for (int hh = 0; hh < g_cfg.nkv; hh++) rope_apply(kv_k + hh*hd, rc, rs);
            memcpy(kslot(l, pos), kv_k, 4*kvd); memcpy(vslot(l, pos), kv_v, 4*kvd);
            attention_plain(l, pos, 1.0f/sqrtf((float)hd));
            matvec(wo[l], NULL, attn, o, d, qd);
            vDSP_vadd(x, 1, o, 1, x, 1, d);
            rmsnorm(x, ln2[l], h, d);
            matvec(wg[l], NULL, h, gate, im, d); matvec(wu[l], NULL, h, up, im, d);
            swiglu(gate, up, act, im);
            matvec(wd[l], NULL, act, m, d, im);
            vDSP_vadd(x, 1, m, 1, x, 1, d);
        }
        rmsnorm(x, final_norm, normed, d);                                            /* final_logits, qwen_infer.c:1585-1599 */
        matvec(head, NULL, normed, logits, V, d);
        if (pos == 0 || pos == n_ids/2 || pos == n_ids - 1) { printf("logits %d", pos); for (int i = 0; i < V; i++) printf(" %.9g", logits[i]); printf("\n"); }
        if (pos >= n_ids - 1) { int am = argmax_v(logits); printf("greedy %d %d\n", pos, am); if (pos + 1 < 4096) ids[pos + 1] = am; }
        /* one more check of rope_head, which rotates without the table: the same numbers as rope_apply */
        if (pos == n_ids - 1) { float a[512], b[512]; for (int i = 0; i < hd; i++) a[i] = b[i] = (float)(i % 7) - 3.0f; rope_head(a, pos); rope_apply(b, rc, rs);
            float worst = 0.0f; for (int i = 0; i < hd; i++) if (fabsf(a[i]-b[i]) > worst) worst = fabsf(a[i]-b[i]); printf("rope_head_vs_apply %.3g\n", worst); }
    }
    return 0;
}
'''


def cut_slices(ref: str, out: str) -> None:
    """Write the lines of qwen_infer.c that the model driver includes into `out`/slice_<name>.inc, after checking
    that each slice still begins where it is expected to."""
    with open(f"{ref}/qwen_infer.c", encoding="utf-8", errors="replace") as f:
        lines = f.read().split("\n")
    for name, (first, last, marker) in MODEL_SLICES.items():
        if marker not in lines[first - 1]:
            raise SystemExit(f"qwen_infer.c:{first} does not hold '{marker}': the slices of make_golden.py want revising")
        with open(f"{out}/slice_{name}.inc", "w") as g:
            g.write("\n".join(lines[first - 1:last]) + "\n")


def write_model_bin(folder: str, path: str) -> None:
    """The folder's tensors as float32 in the order the model driver reads them, behind a header of sizes."""
    import struct
    import numpy as np
    import torch
    from safetensors import safe_open
    cfg = json.load(open(f"{folder}/config.json"))
    with safe_open(f"{folder}/model.safetensors", framework="pt") as f:
        w = {k: f.get_tensor(k).to(torch.float32).numpy() for k in f.keys()}
    nh = cfg["num_attention_heads"]
    hd = cfg.get("head_dim") or cfg["hidden_size"] // nh
    bias = "model.layers.0.self_attn.q_proj.bias" in w
    tied = "lm_head.weight" not in w
    rs = cfg.get("rope_scaling") or {}
    with open(path, "wb") as out:
        out.write(struct.pack("<12i", cfg["num_hidden_layers"], cfg["hidden_size"], nh, cfg["num_key_value_heads"], hd,
                              cfg["intermediate_size"], cfg["vocab_size"], 40000, int(bias), int(tied), int(bool(rs)), 0))
        out.write(struct.pack("<6f", cfg["rope_theta"], cfg["rms_norm_eps"], rs.get("factor", 1.0), rs.get("low_freq_factor", 1.0),
                              rs.get("high_freq_factor", 1.0), rs.get("original_max_position_embeddings", 1.0)))
        order = ["model.embed_tokens.weight"]
        for l in range(cfg["num_hidden_layers"]):
            p = f"model.layers.{l}."
            order += [p + "input_layernorm.weight", p + "self_attn.q_proj.weight", p + "self_attn.k_proj.weight", p + "self_attn.v_proj.weight"]
            if bias:
                order += [p + "self_attn.q_proj.bias", p + "self_attn.k_proj.bias", p + "self_attn.v_proj.bias"]
            order += [p + "self_attn.o_proj.weight", p + "post_attention_layernorm.weight", p + "mlp.gate_proj.weight",
                      p + "mlp.up_proj.weight", p + "mlp.down_proj.weight"]
        order.append("model.norm.weight")
        if not tied:
            order.append("lm_head.weight")
        assert sorted(order) == sorted(w), "the folder holds other tensors than the driver reads"
        for name in order:
            out.write(np.ascontiguousarray(w[name], dtype="<f4").tobytes())


# the sequences of the model goldens: (tiny configuration, seed of the folder, stored type, token ids' seed, tokens, new tokens)
MODEL_CASES = [("A", 21, "float32", 7, 12, 8), ("B", 22, "bfloat16", 8, 19, 6), ("Cfull", 23, "float16", 9, 15, 6)]


def model_case_config(name: str) -> dict:
    """Tiny A and B as they are; C without its window, which the reference does not have (it reads neither
    `use_sliding_window` nor `sliding_window`, qwen_infer.c:1538-1543), but with its frequency scaling and its
    head size given apart from hidden / heads."""
    from helpers import TINY
    if name == "Cfull":
        return dict(TINY["C"][0], use_sliding_window=False)
    return TINY[name][0]


def model_case_folder(root: str, name: str, seed: int, dtype: str) -> str:
    import torch
    from helpers import TINY
    from beglin_b200.weights import write_random_model
    folder = os.path.join(root, f"model_{name}")
    write_random_model(folder, model_case_config(name), seed, dtype=getattr(torch, dtype), **TINY[name[0]][1])
    return folder


def model_case_ids(name: str, ids_seed: int, n: int) -> list:
    import torch
    g = torch.Generator().manual_seed(ids_seed)
    return torch.randint(0, model_case_config(name)["vocab_size"], (n,), generator=g).tolist()


def run_model_driver(tool: str, folder: str, scratch: str, ids: list, n_new: int) -> str:
    write_model_bin(folder, f"{scratch}/model.bin")
    with open(f"{scratch}/tokens.txt", "w") as f:
        f.write(" ".join(str(t) for t in ids))
    return subprocess.run([tool, f"{scratch}/model.bin", f"{scratch}/tokens.txt", str(n_new)], check=True,
                          capture_output=True, text=True).stdout


def build_tools(ref: str, out: str) -> dict:
    """Compile the reference's verify programs from `ref` into `out`; returns name -> executable."""
    tools = {}
    cc = ["gcc", "-O1", "-w", "-I", ref]
    subprocess.run(cc + [f"{ref}/hf_config.c", f"{ref}/hf_config_verify.c", "-o", f"{out}/hf_config_verify", "-lm"], check=True)
    tools["config"] = f"{out}/hf_config_verify"
    subprocess.run(cc + [f"{ref}/safetensors_load.c", f"{ref}/safetensors_quants.c", f"{ref}/hf_config.c",
                         f"{ref}/safetensors_verify.c", "-o", f"{out}/safetensors_verify", "-lm"], check=True)
    tools["checksums"] = f"{out}/safetensors_verify"
    with open(f"{out}/rope_driver.c", "w") as f:
        f.write(ROPE_DRIVER)
    subprocess.run(cc + [f"{out}/rope_driver.c", "-o", f"{out}/rope_driver", "-lm"], check=True)
    tools["rope"] = f"{out}/rope_driver"
    cut_slices(ref, out)
    with open(f"{out}/model_driver.c", "w") as f:
        f.write(MODEL_DRIVER)
    # -ffp-contract=off: no fused multiply-adds, so the float sums are those of the source on every host
    subprocess.run(["gcc", "-O1", "-w", "-ffp-contract=off", "-I", out, "-I", ref, f"{out}/model_driver.c", "-o",
                    f"{out}/model_driver", "-lm"], check=True)
    tools["model"] = f"{out}/model_driver"
    return tools


def run_tools(tools: dict, folder: str) -> dict:
    """The three outputs for one model folder."""
    out = {}
    out["config"] = subprocess.run([tools["config"], f"{folder}/config.json"], check=True, capture_output=True, text=True).stdout
    out["checksums"] = subprocess.run([tools["checksums"], f"{folder}/model.safetensors"], check=True, capture_output=True, text=True).stdout
    cfg = json.load(open(f"{folder}/config.json"))
    rs = cfg.get("rope_scaling")
    if rs:
        hd = cfg.get("head_dim") or cfg["hidden_size"] // cfg["num_attention_heads"]
        args = [cfg["rope_theta"], hd, rs["factor"], rs["low_freq_factor"], rs["high_freq_factor"],
                rs["original_max_position_embeddings"]]
        out["rope_scale"] = subprocess.run([tools["rope"]] + [str(a) for a in args], check=True, capture_output=True, text=True).stdout
    return out


# (name, tiny configuration, seed, stored type): the folders the golden files describe
CASES = [("A", 21, "float32"), ("B", 22, "bfloat16"), ("C", 23, "float16")]


def case_folder(root: str, name: str, seed: int, dtype: str) -> str:
    import torch
    from helpers import TINY
    from beglin_b200.weights import write_random_model
    cfg, init, _ = TINY[name]
    folder = os.path.join(root, f"golden_{name}")
    write_random_model(folder, cfg, seed, dtype=getattr(torch, dtype), **init)
    return folder


def main():
    if len(sys.argv) != 2:
        sys.exit("usage: make_golden.py <path of the reference tree>")
    ref = sys.argv[1]
    with tempfile.TemporaryDirectory() as tmp:
        tools = build_tools(ref, tmp)
        for name, seed, dtype in CASES:
            outs = run_tools(tools, case_folder(tmp, name, seed, dtype))
            for kind, text in outs.items():
                with open(os.path.join(HERE, f"{kind}_{name}.txt"), "w") as f:
                    f.write(text)
                print(f"wrote {kind}_{name}.txt ({len(text)} bytes)")
        for name, seed, dtype, ids_seed, n, n_new in MODEL_CASES:
            text = run_model_driver(tools["model"], model_case_folder(tmp, name, seed, dtype), tmp,
                                    model_case_ids(name, ids_seed, n), n_new)
            with open(os.path.join(HERE, f"model_{name}.txt"), "w") as f:
                f.write(text)
            print(f"wrote model_{name}.txt ({len(text)} bytes)")


if __name__ == "__main__":
    main()
