"""Programs written against the reference's combinator API, shared by the host and GPU tests."""


def user_programs(ops, H=64):
    """The two stacked-LSTM programs as a user of the reference writes them
    (examples/stacked_rnn/stacked_lstm1.py, examples/stacked_rnn/stacked_rnn.py)."""
    def gate_f(w, u, b, x, s):
        y = x @ w + s @ u + b
        return y

    def lstm_cell(h_prev, c_prev, input, ws, us, bs):
        prev_gate = ops.map(lambda x: gate_f(*x, input, h_prev), ops.zip(ws, us, bs))
        gate = ops.map(lambda x: ops.sigmoid(x), prev_gate[:3])
        c = gate[1] * c_prev + gate[0] * ops.tanh(prev_gate[3])
        h = gate[2] * ops.tanh(c)
        return h, c

    def batch_major(embs, Wss, Uss, bss):
        def batched_cell(xs, ws, us, bs):
            return ops.scan(lambda state, x: lstm_cell(*state, x, ws, us, bs), xs,
                            initializer=(ops.zeros(shape=(1, H), device="cpu"), ops.zeros(shape=(1, H), device="cpu")))

        def lstm_layer(xss, Ws, Us, bs):
            hss, css = ops.map(lambda xs: batched_cell(xs, Ws, Us, bs), xss)
            return hss

        return ops.fold(lambda s, param: lstm_layer(s, *param), ops.zip(Wss, Uss, bss), initializer=embs)

    def time_major(embs, Wss, Uss, bss):
        def batched_cell(hs_prev, cs_prev, xs, ws, us, bs):
            return ops.map(lambda x: lstm_cell(*x, ws, us, bs),
                           ops.zip(hs_prev[0:xs.length], cs_prev[0:xs.length], xs))

        def lstm_layer(xss, ws, us, bs):
            init = ops.repeat(ops.zeros(shape=(1, H), device="cpu"), xss[0].length)
            hss, css = ops.scan(lambda state, x: batched_cell(*state, x, ws, us, bs), xss, initializer=(init, init))
            return hss

        return ops.fold(lambda s, param: lstm_layer(s, *param), ops.zip(Wss, Uss, bss), initializer=embs)

    def wrong_gates(embs, Wss, Uss, bss):  # forget gate and input gate swapped: not the LSTM the kernels compute
        def cell(h_prev, c_prev, input, ws, us, bs):
            prev_gate = ops.map(lambda x: gate_f(*x, input, h_prev), ops.zip(ws, us, bs))
            gate = ops.map(lambda x: ops.sigmoid(x), prev_gate[:3])
            c = gate[0] * c_prev + gate[1] * ops.tanh(prev_gate[3])
            return gate[2] * ops.tanh(c), c

        def layer(xss, Ws, Us, bs):
            hss, _ = ops.map(lambda xs: ops.scan(lambda st, x: cell(*st, x, Ws, Us, bs), xs,
                                                 initializer=(ops.zeros(shape=(1, H)), ops.zeros(shape=(1, H)))), xss)
            return hss

        return ops.fold(lambda s, param: layer(s, *param), ops.zip(Wss, Uss, bss), initializer=embs)

    return batch_major, time_major, wrong_gates
