/* The C interface of bitnet.c_b200 (see bn_api.h).  It starts an embedded CPython interpreter on
 * first use, imports the library's bridge module (capi/bridge.py) and turns every call into one
 * call of a bridge function; arrays cross as byte strings.  The repository root is found from the
 * location of this shared object (two folders above capi/), or from $BN_B200_HOME. */
#define PY_SSIZE_T_CLEAN
#define _GNU_SOURCE
#include <Python.h>
#include <dlfcn.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include "bn_api.h"

#ifndef BN_PYTHON_EXECUTABLE
#define BN_PYTHON_EXECUTABLE "python3"
#endif

struct BnModel { PyObject *handle; int vocab, seq_len; };
struct BnSession { BnModel *m; PyObject *handle; float *logits; };
struct BnSampler { PyObject *handle; int vocab; };

static char g_error[1024];
static PyObject *g_bridge;
static int g_started_here;

const char *bn_last_error(void) { return g_error; }

static void set_error(const char *msg) { snprintf(g_error, sizeof(g_error), "%s", msg); }

/* Keep the pending Python exception's message and clear it. */
static void take_py_error(const char *where) {
    PyObject *type = NULL, *value = NULL, *tb = NULL;
    PyErr_Fetch(&type, &value, &tb);
    PyErr_NormalizeException(&type, &value, &tb);
    PyObject *text = value ? PyObject_Str(value) : NULL;
    const char *msg = text ? PyUnicode_AsUTF8(text) : NULL;
    const char *kind = type ? ((PyTypeObject *)type)->tp_name : "error";
    snprintf(g_error, sizeof(g_error), "%s: %s: %s", where, kind, msg ? msg : "(no message)");
    Py_XDECREF(text); Py_XDECREF(type); Py_XDECREF(value); Py_XDECREF(tb);
    PyErr_Clear();
}

static int ensure_bridge(void) {
    if (g_bridge) return 0;
    if (!Py_IsInitialized()) {
        /* the interpreter of the environment the library was built in (its packages hold torch),
         * or the one $BN_B200_PYTHON names */
        const char *exe = getenv("BN_B200_PYTHON");
        if (!exe || !exe[0]) exe = BN_PYTHON_EXECUTABLE;
        PyConfig config;
        PyConfig_InitPythonConfig(&config);
        config.install_signal_handlers = 0;
        PyStatus st = PyConfig_SetBytesString(&config, &config.program_name, exe);
        if (!PyStatus_Exception(st)) st = Py_InitializeFromConfig(&config);
        PyConfig_Clear(&config);
        if (PyStatus_Exception(st)) {
            snprintf(g_error, sizeof(g_error), "cannot start the Python interpreter '%s': %s", exe, st.err_msg ? st.err_msg : "?");
            return -1;
        }
        g_started_here = 1;
    }
    PyGILState_STATE gil = PyGILState_Ensure();
    char root[4096] = "";
    const char *home = getenv("BN_B200_HOME");
    if (home && home[0]) {
        snprintf(root, sizeof(root), "%s", home);
    } else {
        Dl_info info;
        if (dladdr((void *)&ensure_bridge, &info) && info.dli_fname) {
            char *real = realpath(info.dli_fname, NULL);
            if (real) {
                /* .../<root>/bitnet.c_b200/capi/_build/libbitnet_b200.so -> <root> */
                for (int up = 0; up < 4; up++) { char *slash = strrchr(real, '/'); if (slash) *slash = 0; }
                snprintf(root, sizeof(root), "%s", real);
                free(real);
            }
        }
    }
    int rc = -1;
    PyObject *sys_path = PySys_GetObject("path");  /* borrowed */
    PyObject *p = PyUnicode_FromString(root);
    if (sys_path && p && PyList_Insert(sys_path, 0, p) == 0) {
        PyObject *pkg = PyImport_ImportModule("bitnet_c_b200");
        if (pkg) {
            g_bridge = PyImport_ImportModule("bitnet_c_b200.capi.bridge");
            Py_DECREF(pkg);
        }
        if (g_bridge) rc = 0; else take_py_error("importing the library");
    } else {
        set_error("cannot extend sys.path");
    }
    Py_XDECREF(p);
    PyGILState_Release(gil);
    if (g_started_here && rc == 0) PyEval_SaveThread();  /* later calls take the GIL themselves */
    return rc;
}

/* Call bridge.<name>(*args); steals args.  Returns a new reference or NULL (error kept). */
static PyObject *bridge_call(const char *name, PyObject *args) {
    if (!args) { take_py_error(name); return NULL; }
    PyObject *fn = PyObject_GetAttrString(g_bridge, name);
    PyObject *out = fn ? PyObject_CallObject(fn, args) : NULL;
    if (!out) take_py_error(name);
    Py_XDECREF(fn);
    Py_DECREF(args);
    return out;
}

static PyObject *int_bytes(const int *v, int n) { return PyBytes_FromStringAndSize((const char *)v, (Py_ssize_t)n * (Py_ssize_t)sizeof(int)); }

BnModel *bn_model_load(const char *model_dir, const char *dtype, int max_seq_len, const BnCacheParams *cache) {
    if (!model_dir || !dtype) { set_error("bn_model_load: null argument"); return NULL; }
    if (ensure_bridge() != 0) return NULL;
    PyGILState_STATE gil = PyGILState_Ensure();
    BnModel *m = NULL;
    PyObject *h = bridge_call("model_load", Py_BuildValue("(ssiii)", model_dir, dtype, max_seq_len,
                                                          cache ? cache->max_tokens : 0, cache ? cache->max_seqs : 1));
    if (h) {
        PyObject *v = PyObject_GetAttrString(h, "vocab"), *s = PyObject_GetAttrString(h, "seq_len");
        m = (BnModel *)calloc(1, sizeof(*m));
        m->handle = h;
        m->vocab = v ? (int)PyLong_AsLong(v) : 0;
        m->seq_len = s ? (int)PyLong_AsLong(s) : 0;
        Py_XDECREF(v); Py_XDECREF(s);
    }
    PyGILState_Release(gil);
    return m;
}

void bn_model_free(BnModel *m) {
    if (!m) return;
    PyGILState_STATE gil = PyGILState_Ensure();
    Py_XDECREF(m->handle);
    PyGILState_Release(gil);
    free(m);
}

int bn_model_vocab_size(const BnModel *m) { return m ? m->vocab : -1; }
int bn_model_seq_len(const BnModel *m) { return m ? m->seq_len : -1; }

BnSession *bn_session_create(BnModel *m) {
    if (!m) { set_error("bn_session_create: null model"); return NULL; }
    PyGILState_STATE gil = PyGILState_Ensure();
    BnSession *s = NULL;
    PyObject *h = bridge_call("session_create", Py_BuildValue("(O)", m->handle));
    if (h) {
        s = (BnSession *)calloc(1, sizeof(*s));
        s->m = m; s->handle = h;
        s->logits = (float *)malloc((size_t)m->vocab * sizeof(float));
    }
    PyGILState_Release(gil);
    return s;
}

static int session_method(BnSession *s, const char *name) {
    PyGILState_STATE gil = PyGILState_Ensure();
    PyObject *r = PyObject_CallMethod(s->handle, name, NULL);
    int rc = -1;
    if (r) { rc = PyLong_Check(r) ? (int)PyLong_AsLong(r) : 0; Py_DECREF(r); } else take_py_error(name);
    PyGILState_Release(gil);
    return rc;
}

void bn_session_free(BnSession *s) {
    if (!s) return;
    session_method(s, "close");
    PyGILState_STATE gil = PyGILState_Ensure();
    Py_XDECREF(s->handle);
    PyGILState_Release(gil);
    free(s->logits);
    free(s);
}

int bn_session_reset(BnSession *s) { return s ? session_method(s, "reset") : -1; }
int bn_session_pos(const BnSession *s) { return s ? session_method((BnSession *)s, "pos") : -1; }

/* want: 0 none, 1 last, 2 all; copies the returned floats to dst (count floats expected). */
static int run_prefill(BnModel *m, BnSession *s, const int *tokens, int n, int pos0, int no_prefill, int want, float *dst,
                       size_t count) {
    if (!m || !s || !tokens || n <= 0) { set_error("prefill: bad argument"); return -1; }
    PyGILState_STATE gil = PyGILState_Ensure();
    int rc = -1;
    PyObject *r = bridge_call("prefill", Py_BuildValue("(OONiii)", m->handle, s->handle, int_bytes(tokens, n), pos0,
                                                       no_prefill, want));
    if (r) {
        char *data; Py_ssize_t len;
        if (PyBytes_AsStringAndSize(r, &data, &len) == 0 && (size_t)len == count * sizeof(float)) {
            if (count) memcpy(dst, data, (size_t)len);
            rc = 0;
        } else {
            set_error("prefill: the engine returned logits of an unexpected size");
        }
        Py_DECREF(r);
    }
    PyGILState_Release(gil);
    return rc;
}

const float *bn_prefill(BnModel *m, BnSession *s, const int *tokens, int n_tokens, int pos0, int no_prefill) {
    if (!m || !s) { set_error("bn_prefill: null argument"); return NULL; }
    return run_prefill(m, s, tokens, n_tokens, pos0, no_prefill, 1, s->logits, (size_t)m->vocab) == 0 ? s->logits : NULL;
}

int bn_prefill_no_logits(BnModel *m, BnSession *s, const int *tokens, int n_tokens, int pos0, int no_prefill) {
    return run_prefill(m, s, tokens, n_tokens, pos0, no_prefill, 0, NULL, 0);
}

const float *bn_transformer_forward(BnModel *m, BnSession *s, int token, int pos) {
    return bn_prefill(m, s, &token, 1, pos, 0);
}

int bn_transformer_prefill_all(BnModel *m, BnSession *s, const int *tokens, int n_tokens, int pos0, float *all_logits) {
    if (!m || !all_logits) { set_error("bn_transformer_prefill_all: null argument"); return -1; }
    return run_prefill(m, s, tokens, n_tokens, pos0, 0, 2, all_logits, (size_t)n_tokens * (size_t)m->vocab);
}

int bn_step(BnModel *m, BnSession *const *sessions, int n_sessions, const int *n_new, const int *tokens, float *logits_out) {
    if (!m || !sessions || n_sessions <= 0 || !n_new || !tokens) { set_error("bn_step: bad argument"); return -1; }
    int total = 0;
    for (int i = 0; i < n_sessions; i++) total += n_new[i];
    PyGILState_STATE gil = PyGILState_Ensure();
    int rc = -1;
    PyObject *list = PyList_New(n_sessions);
    for (int i = 0; i < n_sessions; i++) { Py_INCREF(sessions[i]->handle); PyList_SET_ITEM(list, i, sessions[i]->handle); }
    PyObject *r = bridge_call("step", Py_BuildValue("(ONNNi)", m->handle, list, int_bytes(n_new, n_sessions),
                                                    int_bytes(tokens, total), logits_out ? 1 : 0));
    if (r) {
        char *data; Py_ssize_t len;
        size_t want = logits_out ? (size_t)n_sessions * (size_t)m->vocab * sizeof(float) : 0;
        if (PyBytes_AsStringAndSize(r, &data, &len) == 0 && (size_t)len == want) {
            if (want) memcpy(logits_out, data, want);
            rc = 0;
        } else {
            set_error("bn_step: the engine returned logits of an unexpected size");
        }
        Py_DECREF(r);
    }
    PyGILState_Release(gil);
    return rc;
}

BnSampler *bn_sampler_create(int vocab_size, const BnSamplerParams *p) {
    if (vocab_size <= 0 || !p) { set_error("bn_sampler_create: bad argument"); return NULL; }
    if (ensure_bridge() != 0) return NULL;
    PyGILState_STATE gil = PyGILState_Ensure();
    BnSampler *s = NULL;
    PyObject *h = bridge_call("sampler_create", Py_BuildValue("(idddiK)", vocab_size, (double)p->temperature, (double)p->topp,
                                                              (double)(p->repeat_penalty > 0 ? p->repeat_penalty : 1.0f),
                                                              p->repeat_window, p->seed));
    if (h) { s = (BnSampler *)calloc(1, sizeof(*s)); s->handle = h; s->vocab = vocab_size; }
    PyGILState_Release(gil);
    return s;
}

void bn_sampler_free(BnSampler *s) {
    if (!s) return;
    PyGILState_STATE gil = PyGILState_Ensure();
    Py_XDECREF(s->handle);
    PyGILState_Release(gil);
    free(s);
}

void bn_sampler_accept(BnSampler *s, int token) {
    if (!s) return;
    PyGILState_STATE gil = PyGILState_Ensure();
    PyObject *r = PyObject_CallMethod(s->handle, "accept", "i", token);
    if (!r) take_py_error("bn_sampler_accept");
    Py_XDECREF(r);
    PyGILState_Release(gil);
}

int bn_sampler_sample(BnSampler *s, const float *logits) {
    if (!s || !logits) { set_error("bn_sampler_sample: null argument"); return -1; }
    PyGILState_STATE gil = PyGILState_Ensure();
    int tok = -1;
    PyObject *r = PyObject_CallMethod(s->handle, "sample", "y#", (const char *)logits, (Py_ssize_t)s->vocab * (Py_ssize_t)sizeof(float));
    if (r) { tok = (int)PyLong_AsLong(r); Py_DECREF(r); } else take_py_error("bn_sampler_sample");
    PyGILState_Release(gil);
    return tok;
}

int bn_generate_batch(BnModel *m, const int *const *prompts, const int *prompt_lens, int n_prompts, int max_new_tokens,
                      const BnSamplerParams *sp, const int *stop_ids, int n_stop_ids, int *const *out_tokens, int *out_counts) {
    if (!m || !prompts || !prompt_lens || n_prompts <= 0 || !sp || !out_tokens || !out_counts) {
        set_error("bn_generate_batch: bad argument");
        return -1;
    }
    PyGILState_STATE gil = PyGILState_Ensure();
    int rc = -1;
    PyObject *list = PyList_New(n_prompts);
    for (int i = 0; i < n_prompts; i++) PyList_SET_ITEM(list, i, int_bytes(prompts[i], prompt_lens[i]));
    PyObject *r = bridge_call("generate_batch", Py_BuildValue("(ONidddiKN)", m->handle, list, max_new_tokens, (double)sp->temperature,
                                                              (double)sp->topp, (double)(sp->repeat_penalty > 0 ? sp->repeat_penalty : 1.0f),
                                                              sp->repeat_window, sp->seed, int_bytes(stop_ids, stop_ids ? n_stop_ids : 0)));
    if (r && PyList_Check(r) && PyList_GET_SIZE(r) == n_prompts) {
        rc = 0;
        for (int i = 0; i < n_prompts; i++) {
            char *data; Py_ssize_t len;
            if (PyBytes_AsStringAndSize(PyList_GET_ITEM(r, i), &data, &len) != 0 || len > (Py_ssize_t)max_new_tokens * (Py_ssize_t)sizeof(int)) {
                set_error("bn_generate_batch: the engine returned more tokens than asked for");
                rc = -1;
                break;
            }
            memcpy(out_tokens[i], data, (size_t)len);
            out_counts[i] = (int)(len / (Py_ssize_t)sizeof(int));
        }
    }
    Py_XDECREF(r);
    PyGILState_Release(gil);
    return rc;
}
