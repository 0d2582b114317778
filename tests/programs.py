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


def attention_program(ops, blk, d, scale=None):
    """Blockwise attention with the online-softmax carry (examples/flash_attention/flash_attention.py),
    the carry started in (max, sum, out) order."""
    def attn_func(prev_maxes, prev_sums, prev_out, query, key, value):
        attn_weights = query @ key.T
        if scale is not None:
            attn_weights = attn_weights * scale
        cur_maxes = ops.max(attn_weights, dim=-1, keepdim=True)
        exp_weights = ops.exp(attn_weights - cur_maxes)
        exp_values = exp_weights @ value
        cur_sums = ops.sum(exp_weights, dim=-1, keepdim=True)
        new_maxes = ops.maximum(cur_maxes, prev_maxes)
        renorm_prev = ops.exp(prev_maxes - new_maxes)
        renorm_cur = ops.exp(cur_maxes - new_maxes)
        new_sums = renorm_prev * prev_sums + renorm_cur * cur_sums
        o = (prev_out * prev_sums * renorm_prev + renorm_cur * exp_values) / new_sums
        return new_maxes, new_sums, o

    def per_block_func(query, ks, vs):
        init_sum = ops.zeros(shape=(blk, 1), device="cpu")
        init_max = ops.full(shape=(blk, 1), fill_value=-3.4028234663852886e38, device="cpu")
        init_o = ops.zeros(shape=(blk, d), device="cpu")
        _, _, o = ops.reduce(lambda state, kvs: attn_func(*state, query, *kvs), ops.zip(ks, vs),
                             initializer=(init_max, init_sum, init_o))
        return o

    def per_head_func(qs, ks, vs):
        return ops.map(lambda q_: per_block_func(q_, ks, vs), qs)

    def flash_attention(qsss, ksss, vsss):
        return ops.map(lambda xss: ops.map(lambda xs: per_head_func(*xs), ops.zip(*xss)), ops.zip(qsss, ksss, vsss))

    return flash_attention


def dilated_program(ops, H=64):
    """The stacked dilated LSTM (examples/dilated_rnn/dilated_rnn.py): layer i scans 2**i interleaved
    sub-sequences."""
    def gate_f(w, u, b, x, s):
        return x @ w + s @ u + b

    def lstm_cell(h_prev, c_prev, input, ws, us, bs):
        prev_gate = ops.map(lambda x: gate_f(*x, input, h_prev), ops.zip(ws, us, bs))
        gate = ops.map(lambda x: ops.sigmoid(x), prev_gate[:3])
        c = gate[1] * c_prev + gate[0] * ops.tanh(prev_gate[3])
        h = gate[2] * ops.tanh(c)
        return h, c

    def dilated_layer(state, itr, Ws, Us, bs):
        zeros = ops.zeros(shape=(1, H), device="cpu", dtype="float")
        h, _ = ops.dilated_map(
            lambda xs: ops.scan(lambda s, x: lstm_cell(*s, x, Ws, Us, bs), xs, initializer=(zeros, zeros)),
            state, dilation=2 ** itr)
        return h

    def model(embs, Wss, Uss, bss):
        itrs = ops.enumerate(Wss, Uss, bss)
        return ops.map(lambda xs: ops.fold(lambda s, x: dilated_layer(s, *x), itrs, initializer=xs), embs)

    return model


def grid_program(ops, H):
    """The stacked grid RNN as the example writes it (examples/grid_rnn/grid_rnn.py:42-146): a tanh
    cell per direction on the concatenated (state from above, state from the left)."""
    def vanilla_cell(state, cur, i2h, h2h, bias):
        h = ops.tanh(cur @ i2h + state @ h2h + bias)
        return h

    def grid_cell(state, cur_input, block_params):
        _, state_y = state
        state_x, (x_t, y_t) = cur_input
        rnn_param_x, rnn_param_y = block_params
        s = ops.cat([state_x, state_y], dim=1)
        h_x = vanilla_cell(x_t, s, *rnn_param_x)
        h_y = vanilla_cell(y_t, s, *rnn_param_y)
        return h_x, h_y

    def direction_y(state, cur_input, block_params):
        state_xs, _ = state
        zero = ops.zeros(shape=(1, H), device="cpu")
        ys = ops.scan(lambda s, x: grid_cell(s, x, block_params), ops.zip(state_xs, ops.zip(*cur_input)),
                      initializer=(zero, zero))
        return ys

    def direction_x(state, block_params):
        zeros = ops.repeat(ops.zeros(shape=(1, H), device="cpu"), len(state[0][0]))
        ys1, ys2 = ops.scan(lambda s, x: direction_y(s, x, block_params), state, initializer=(zeros, zeros))
        return ops.zip(ys1, ys2)

    def stacked_grid_rnns(src_encs, trg_encs, stacked_params):
        return ops.fold(lambda inputs, params: direction_x(inputs, params), stacked_params,
                        initializer=ops.zip(*ops.product(src_encs, trg_encs)))

    def model(src_encs, trg_encs, stacked_params):
        return ops.map(lambda x: stacked_grid_rnns(*x, stacked_params), ops.zip(src_encs, trg_encs))

    def wrong_state(src_encs, trg_encs, stacked_params):  # both cells fed the state from above twice
        def bad_cell(state, cur_input, block_params):
            state_x, (x_t, y_t) = cur_input
            s = ops.cat([state_x, state_x], dim=1)
            return vanilla_cell(x_t, s, *block_params[0]), vanilla_cell(y_t, s, *block_params[1])

        def bad_y(state, cur_input, block_params):
            zero = ops.zeros(shape=(1, H), device="cpu")
            return ops.scan(lambda s, x: bad_cell(s, x, block_params), ops.zip(state[0], ops.zip(*cur_input)),
                            initializer=(zero, zero))

        def bad_x(state, block_params):
            zeros = ops.repeat(ops.zeros(shape=(1, H), device="cpu"), len(state[0][0]))
            ys1, ys2 = ops.scan(lambda s, x: bad_y(s, x, block_params), state, initializer=(zeros, zeros))
            return ops.zip(ys1, ys2)

        return ops.map(lambda x: ops.fold(lambda i, p: bad_x(i, p), stacked_params,
                                          initializer=ops.zip(*ops.product(*x))), ops.zip(src_encs, trg_encs))

    return model, wrong_state
