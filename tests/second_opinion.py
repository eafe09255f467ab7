"""A second, independently written restatement of the reference's numerics references, used only
to cross-check the oracle (oracle/ref_order.c and oracle/oracle.py share no code with this file).

Written from the reference's own text, one numpy float32 scalar operation per line of it:
  * `sdpa_expected_output`: src/kernel/library/attention.zig:473-509 (`expectedOutput`): scores
    with the running maximum, the sum of exponentials, then the weighted sum with the weight
    recomputed per key; scale = 1 / sqrt(qk);
  * `row_softmax`: normalization.zig:300-310 (exp(value - row_max) summed in column order) and the
    distribution kernel around it;
  * `row_layer_norm`: normalization.zig:560-590: mean = sum / cols, variance from a second fold of
    (value - mean)^2, `variance + epsilon`, sqrt, (value - mean) / root;
  * `row_rms_norm`: normalization.zig:372-398: mean square + epsilon, sqrt, value / root, * weight;
  * `gelu_tanh`: src/kernel/library/elementwise.zig:125-135, operation by operation;
  * `dot_serial`: src/preparation/kernelization/lowering/dot.zig:2049-2115: acc = acc + a*b over k.
Python loops over numpy float32 scalars: slow, meant for the reference's own tiny specs
(attention.zig:464-471: batch 2, queries 2, keys 3, qk 2, value 2) and a few dozen elements.
"""
import numpy as np

F = np.float32


def sdpa_expected_output(queries, keys, values, batch, query, value, n_queries, n_keys, qk, n_value, causal=False):
    scores = [F(0)] * n_keys
    scale = F(1.0 / np.sqrt(float(qk)))
    max_score = F(-np.inf)
    for key in range(n_keys):
        dot = F(0.0)
        for feature in range(qk):
            query_offset = batch * n_queries * qk + query * qk + feature
            key_offset = batch * n_keys * qk + key * qk + feature
            dot = F(dot + F(queries[query_offset] * keys[key_offset]))
        score = F(dot * scale)
        if causal and key > query:
            score = F(-np.inf)
        scores[key] = score
        if score > max_score:
            max_score = score
    denominator = F(0.0)
    for score in scores:
        denominator = F(denominator + np.exp(F(score - max_score)))
    total = F(0.0)
    for key in range(n_keys):
        weight = F(np.exp(F(scores[key] - max_score)) / denominator)
        value_offset = batch * n_keys * n_value + key * n_value + value
        total = F(total + F(weight * values[value_offset]))
    return total


def sdpa(queries, keys, values, causal=False):
    """[batch, queries, qk] x [batch, keys, qk] x [batch, keys, value] -> [batch, queries, value]"""
    b, nq, qk = queries.shape
    nk, nv = keys.shape[1], values.shape[2]
    q, k, v = (np.ascontiguousarray(a, F).reshape(-1) for a in (queries, keys, values))
    out = np.zeros((b, nq, nv), F)
    for bi in range(b):
        for qi in range(nq):
            for vi in range(nv):
                out[bi, qi, vi] = sdpa_expected_output(q, k, v, bi, qi, vi, nq, nk, qk, nv, causal)
    return out


def row_softmax(row):
    row_max = F(-np.inf)
    for value in row:
        row_max = value if value > row_max else row_max
    total = F(0.0)
    for value in row:
        total = F(total + np.exp(F(value - row_max)))
    return np.array([F(np.exp(F(value - row_max)) / total) for value in row], F)


def row_layer_norm(row, epsilon):
    cols = F(len(row))
    total = F(0.0)
    for value in row:
        total = F(total + value)
    mean = F(total / cols)
    variance_sum = F(0.0)
    for value in row:
        centred = F(value - mean)
        variance_sum = F(variance_sum + F(centred * centred))
    variance = F(variance_sum / cols)
    root = F(np.sqrt(F(variance + F(epsilon))))
    return np.array([F(F(value - mean) / root) for value in row], F)


def row_rms_norm(row, weight, epsilon):
    cols = F(len(row))
    sum_squares = F(0.0)
    for value in row:
        sum_squares = F(sum_squares + F(value * value))
    root = F(np.sqrt(F(F(sum_squares / cols) + F(epsilon))))
    return np.array([F(F(value / root) * w) for value, w in zip(row, weight)], F)


def gelu_tanh(value):
    value = F(value)
    square = F(value * value)
    cube = F(square * value)
    cubic = F(cube * F(0.044715))
    shifted = F(value + cubic)
    scaled = F(shifted * F(0.7978845608028654))
    smooth = F(np.tanh(scaled))
    gate = F(smooth + F(1.0))
    half_value = F(value * F(0.5))
    return F(half_value * gate)


def dot_serial(lhs, rhs):
    """[m, k] x [k, n] -> [m, n], every element folded over k in increasing order"""
    m, k = lhs.shape
    n = rhs.shape[1]
    out = np.zeros((m, n), F)
    for i in range(m):
        for j in range(n):
            acc = F(0.0)
            for kk in range(k):
                acc = F(acc + F(F(lhs[i, kk]) * F(rhs[kk, j])))
            out[i, j] = acc
    return out


def mlp_rms(x, w1, b1, w2, b2, g, epsilon):
    hidden = dot_serial(x, w1)
    act = np.array([[gelu_tanh(F(h + b)) for h, b in zip(row, b1)] for row in hidden], F)
    y = dot_serial(act, w2)
    y = np.array([[F(v + b) for v, b in zip(row, b2)] for row in y], F)
    return np.stack([row_rms_norm(row, g, epsilon) for row in y])
