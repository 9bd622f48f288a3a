"""Attention, recurrent and preprocessing layers against plain-PyTorch references."""

import numpy as np
import pytest
import torch

import keras_b200 as keras
from keras_b200 import layers


def test_multi_head_attention_matches_manual_attention():
    torch.manual_seed(0)
    mha = layers.MultiHeadAttention(num_heads=2, key_dim=4)
    x = np.random.RandomState(0).randn(2, 5, 8).astype("float32")
    y, scores = mha(x, x, return_attention_scores=True, use_causal_mask=True)
    q = torch.einsum("abc,cde->abde", torch.tensor(x), mha.query_dense.kernel.value) + mha.query_dense.bias.value
    k = torch.einsum("abc,cde->abde", torch.tensor(x), mha.key_dense.kernel.value) + mha.key_dense.bias.value
    v = torch.einsum("abc,cde->abde", torch.tensor(x), mha.value_dense.kernel.value) + mha.value_dense.bias.value
    logits = torch.einsum("btnh,bsnh->bnts", q, k) / 2.0
    logits = logits.masked_fill(~torch.ones(5, 5, dtype=torch.bool).tril(), -1e9)
    p = torch.softmax(logits, -1)
    o = torch.einsum("bnts,bsnh->btnh", p, v)
    ref = torch.einsum("btnh,nhd->btd", o, mha.output_dense.kernel.value) + mha.output_dense.bias.value
    np.testing.assert_allclose(y.detach().numpy(), ref.detach().numpy(), rtol=1e-4, atol=1e-5)
    np.testing.assert_allclose(scores.detach().numpy(), p.detach().numpy(), rtol=1e-4, atol=1e-6)
    fast = mha(x, x, use_causal_mask=True)  # fused scaled-dot-product path
    np.testing.assert_allclose(fast.detach().numpy(), ref.detach().numpy(), rtol=1e-4, atol=1e-5)
    assert [v.path.split("/", 1)[1] for v in mha.weights] == ["query/kernel", "query/bias", "key/kernel", "key/bias", "value/kernel", "value/bias",
                                                             "attention_output/kernel", "attention_output/bias"]


def test_grouped_query_attention_paths_agree_and_mask():
    gqa = layers.GroupedQueryAttention(head_dim=4, num_query_heads=4, num_key_value_heads=2)
    x = np.random.RandomState(1).randn(2, 6, 8).astype("float32")
    mask = np.tril(np.ones((2, 6, 6), bool))
    fast = gqa(x, x, attention_mask=mask)
    slow, scores = gqa(x, x, attention_mask=mask, return_attention_scores=True)
    np.testing.assert_allclose(fast.detach().numpy(), slow.detach().numpy(), rtol=1e-4, atol=1e-5)
    assert float(scores[0, 0, 0, 1]) == 0.0


def test_lstm_and_gru_match_torch_modules():
    x = np.random.RandomState(2).randn(3, 7, 5).astype("float32")
    lstm = layers.LSTM(6, return_sequences=True)
    lstm.build((3, 7, 5))
    t = torch.nn.LSTM(5, 6, batch_first=True)
    with torch.no_grad():
        t.weight_ih_l0.copy_(lstm.cell.kernel.value.T)
        t.weight_hh_l0.copy_(lstm.cell.recurrent_kernel.value.T)
        t.bias_ih_l0.copy_(lstm.cell.bias.value)
        t.bias_hh_l0.zero_()
    np.testing.assert_allclose(lstm(x).detach().numpy(), t(torch.tensor(x))[0].detach().numpy(), rtol=1e-4, atol=1e-5)
    gru = layers.GRU(6, return_sequences=True)
    gru.build((3, 7, 5))
    g = torch.nn.GRU(5, 6, batch_first=True)
    u = 6
    k, rk, b = gru.cell.kernel.value, gru.cell.recurrent_kernel.value, gru.cell.bias.value

    def zrh_to_rzn(w):  # keras gate order z, r, h -> torch r, z, n
        return torch.cat([w[..., u:2 * u], w[..., :u], w[..., 2 * u:]], dim=-1)

    with torch.no_grad():
        g.weight_ih_l0.copy_(zrh_to_rzn(k).T)
        g.weight_hh_l0.copy_(zrh_to_rzn(rk).T)
        g.bias_ih_l0.copy_(zrh_to_rzn(b[0]))
        g.bias_hh_l0.copy_(zrh_to_rzn(b[1]))
    np.testing.assert_allclose(gru(x).detach().numpy(), g(torch.tensor(x))[0].detach().numpy(), rtol=1e-4, atol=1e-5)
    # generic time loop (masked) equals the hoisted path on unmasked steps and freezes state on masked ones
    mask = np.array([[1] * 7, [1, 1, 1, 0, 0, 0, 0], [1] * 5 + [0, 0]], dtype=bool)
    ym = lstm(x, mask=mask)
    np.testing.assert_allclose(ym[1, 2].detach().numpy(), ym[1, 6].detach().numpy())
    np.testing.assert_allclose(ym[0].detach().numpy(), lstm(x)[0].detach().numpy(), rtol=1e-5, atol=1e-6)


def test_bidirectional_and_saving_roundtrip(tmp_path):
    x = np.random.RandomState(3).randn(4, 6, 3).astype("float32")
    inp = keras.Input((6, 3))
    h = layers.Bidirectional(layers.GRU(4, return_sequences=True))(inp)
    h = layers.TimeDistributed(layers.Dense(2))(h)
    out = layers.SimpleRNN(3)(h)
    m = keras.Model(inp, out)
    path = str(tmp_path / "rnn.keras")
    m.save(path)
    m2 = keras.saving.load_model(path)
    np.testing.assert_allclose(m.predict(x, verbose=0), m2.predict(x, verbose=0), rtol=1e-6)


def test_normalization_adapt_and_text_vectorization():
    x = (np.random.RandomState(4).randn(200, 3) * [1, 5, 0.1] + [0, 10, -3]).astype("float32")
    n = layers.Normalization()
    n.adapt([x[:64], x[64:]])
    y = keras.ops.convert_to_numpy(n(x))
    np.testing.assert_allclose(y.mean(0), 0, atol=1e-4)
    np.testing.assert_allclose(y.std(0), 1, atol=1e-3)
    tv = layers.TextVectorization(max_tokens=8, output_sequence_length=4)
    tv.adapt(["the cat sat", "the dog sat down", "the end"])
    assert tv.get_vocabulary()[:4] == ["", "[UNK]", "the", "sat"]
    out = tv(["the cat flew", "sat"])
    assert out.shape == (2, 4) and out[0, 0] == 2 and out[0, 2] == 1 and out[1, 1] == 0
    sl = layers.StringLookup(vocabulary=["a", "b"], output_mode="one_hot")
    np.testing.assert_array_equal(keras.ops.convert_to_numpy(sl(np.array(["b", "zzz"]))), [[0, 0, 1], [1, 0, 0]])


def test_image_augmentation_geometry_and_boxes():
    img = np.arange(16, dtype="float32").reshape(1, 4, 4, 1)
    rot = layers.RandomRotation((0.25, 0.25), fill_mode="constant")
    np.testing.assert_allclose(keras.ops.convert_to_numpy(rot(img, training=True))[0, :, :, 0], np.rot90(img[0, :, :, 0]), atol=1e-4)
    np.testing.assert_allclose(keras.ops.convert_to_numpy(rot(img, training=False)), img)
    flip = layers.RandomFlip("horizontal", bounding_box_format="xyxy", seed=1)
    data = {"images": np.zeros((8, 10, 20, 3), "float32"),
            "bounding_boxes": {"boxes": np.tile(np.array([[[2.0, 1.0, 6.0, 5.0]]], "float32"), (8, 1, 1)), "labels": np.zeros((8, 1), "int64")}}
    out = flip(data, training=True)["bounding_boxes"]["boxes"].numpy()
    assert set(map(tuple, out[:, 0].tolist())) <= {(2.0, 1.0, 6.0, 5.0), (14.0, 1.0, 18.0, 5.0)}
    crop = layers.CenterCrop(4, 4)
    assert tuple(crop(np.zeros((2, 8, 8, 3), "float32")).shape) == (2, 4, 4, 3)
    mix = layers.MixUp(seed=0)({"images": np.random.rand(4, 8, 8, 3).astype("float32"), "labels": np.eye(4, dtype="float32")})
    np.testing.assert_allclose(mix["labels"].sum(1).numpy(), 1.0, rtol=1e-6)
