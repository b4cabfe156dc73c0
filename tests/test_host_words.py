"""CPU tests of the C++ host side: the words machine (grammar, builtins, base words), the
tensor facade on host tensors, the generated model scripts, and -- when the reference checkout
is on this machine -- the reference's own init.words / train.words running through this machine."""
import os
import re

import numpy as np
import pytest

from blackriver_b200 import host, words

REF = os.path.join(os.environ.get("BLACKRIVER_REFERENCE", os.path.join(os.sep, "root", "reference")), "bloomz-7b")


@pytest.fixture()
def env():
    e = host.Env(4)
    yield e
    e.close()


def test_abi_symbols_of_host_library():
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    txt = open(os.path.join(root, "include", "br_host.h")).read()
    names = re.findall(r"^BRH_API[^;(]*?\b(brh_\w+)\s*\(", txt, flags=re.M)
    assert len(names) >= 20 and set(names) == set(host.SIGNATURES)
    for n in names:
        assert hasattr(host.lib(), n)


def test_arithmetic_and_stack_words(env):
    env.execute("7 2 - 3 * 4 /")
    assert env.pop_number() == 3.75
    env.execute("7 2 //")
    assert env.pop_number() == 3
    env.execute("1 2 swap")
    assert (env.pop_number(), env.pop_number()) == (1, 2)
    env.execute("1 2 3 rot")                 # ( c b a -- b a c )
    assert [env.pop_number() for _ in range(3)] == [1, 3, 2]
    env.execute("1 2 dup2")                  # the pair three times over
    assert env.stack_size == 6
    env.clear_stack()
    env.execute('"ab" "cd" |')
    assert env.pop_string() == "abcd"
    env.execute("-3 1e-05 2.5 ture false")
    assert [env.pop_number() for _ in range(5)] == [0, 1, 2.5, 1e-05, -3]
    env.execute("null")
    assert env.pop_string() == ""


def test_separators_comments_strings(env):
    env.execute('( 1 2 ) { + }   ; a comment 99\n "a ; b" \'x y\' $name')
    assert env.pop_string() == "$name"
    assert env.pop_string() == "x y"
    assert env.pop_string() == "a ; b"
    assert env.pop_number() == 3
    with pytest.raises(host.HostError):
        env.execute('"unterminated')


def test_hash_builtins_and_tables(env):
    env.execute('5 "k" !  "k" @  "k" @ +')
    assert env.pop_number() == 10
    env.execute('##')
    assert env.pop_number() == 0
    env.execute('2 #  9 "k" !  "k" @  ##  0 #  "k" @')
    assert [env.pop_number() for _ in range(3)] == [5, 2, 9]
    env.execute('"k" !!')
    assert not env.has("k")
    with pytest.raises(host.HostError):
        env.execute('"k" @')
    with pytest.raises(host.HostError):
        env.execute("9 #")
    env.execute('3 $batch !  $batch @')
    assert env.pop_number() == 3


def test_user_words_lists_and_errors(env):
    env.execute("%def twice dup + %end  %def quad twice twice %end  3 quad")
    assert env.pop_number() == 12
    env.execute("[ 4 5 6 ]")
    assert [env.pop_number() for _ in range(4)] == [3, 6, 5, 4]
    env.execute("[ ]")
    assert env.pop_number() == 0
    for bad in ("%def twice 1 %end", "%def 9x 1 %end", "%def a 1", "%end", "[ 1 2", "1 ]", "%def b %def c %end %end",
                "undefined_word"):
        with pytest.raises(host.HostError):
            env.execute(bad)
    env.clear_stack()
    with pytest.raises(host.HostError):
        env.execute("drop")                  # stack underflow


def test_host_tensor_storage_ops(env, tmp_path):
    env.execute('2 3 4 3 "cpu" "float" op.create "t" !  "t" @ 2.5 op.fill')
    assert env.tensor_info("t") == {**env.tensor_info("t"), "cuda": False, "dtype": 0, "shape": (2, 3, 4)}
    assert (env.read("t") == 2.5).all()
    a = np.arange(24, dtype=np.float32).reshape(2, 3, 4)
    env.write("t", a)
    env.execute('"t" @ 4 0 5 2 op.view "v" !')   # one open dimension: (24-4)/5 = 4
    assert env.tensor_info("v")["shape"] == (4, 5)
    assert (env.read("v") == a.reshape(-1)[4:].reshape(4, 5)).all()
    env.execute('24 1 "cpu" "float" op.create "u" !  "u" @ "t" @ op.copy  "t" @ op.zero')
    assert (env.read("u") == a.reshape(-1)).all() and (env.read("t") == 0).all()
    f = str(tmp_path / "u.bin")
    env.execute(f'"u" @ "{f}" io.save  "t" @ "{f}" io.load')
    assert (env.read("t") == a).all()
    env.execute('6 1 "cpu" "int" op.create "i" !')
    env.write("i", np.arange(6, dtype=np.int32))
    assert env.read("i").tolist() == list(range(6))
    with pytest.raises(host.HostError):
        env.execute('"t" @ 20 5 1 op.view')       # reaches outside the tensor
    with pytest.raises(host.HostError):
        env.execute('"t" @ "u" @ "t" @ op.add')   # host tensors carry no math


def test_generated_scripts_define_the_driver_words(env):
    env.execute(words.init_words(hidden=64, heads=4, vocab=96, dtype="float"))
    env.execute(words.train_words())
    env.execute('"cpu" $DEVICE !  create_layer_weight create_layer_grad zero_layer_grad')
    assert env.tensor_info("query_key_value.weight")["shape"] == (192, 64)
    assert env.tensor_info("key.weight")["shape"] == (64, 64)
    w = np.arange(192 * 64, dtype=np.float32).reshape(192, 64)
    env.write("query_key_value.weight", w)
    assert (env.read("value.weight") == w[128:]).all()          # rows 2H..3H-1 are the value projection
    assert (env.read("dense_4h_to_h.weight_g") == 0).all()
    assert env.get_number("HEAD_HIDDEN") == 16


@pytest.mark.skipif(not os.path.exists(os.path.join(REF, "init.words")), reason="reference scripts not on this machine")
def test_reference_scripts_run_on_this_machine(env):
    init = open(os.path.join(REF, "init.words")).read()
    train = open(os.path.join(REF, "train.words")).read()
    # shrink the model constants so that host tensors stay tiny; nothing else is edited
    init = init.replace("250880 ", "96 ", 1).replace("4096 ", "64 ", 1).replace("32 ", "4 ", 1).replace("128 ", "16 ", 1)
    prog = env.build(init)                 # compiled once, run per hash table (train_bloom.cpp:128-148)
    env.run(prog)
    env.execute(train)                     # definitions only, as the driver does first
    assert env.get_number("HIDDEN_SIZE") == 64 and env.get_number("HIDDEN_SIZE_x4") == 256
    env.change(1)
    env.run(prog)
    env.free_program(prog)
    env.execute('"cpu" $DEVICE !  create_layer_input create_layer_weight create_layer_grad zero_layer_grad')
    assert env.tensor_info("query.weight")["shape"] == (64, 64)
    assert env.tensor_info("dense_h_to_4h.weight_g")["shape"] == (256, 64)
    assert env.tensor_info("_xinput_")["shape"] == (8192, 64)


def test_new_words_without_a_device():
    """The extension words exist in the words machine and fail cleanly (an error, not a crash) where they need the
    device context; op.kernel_status answers 0 when nothing has been booted."""
    from blackriver_b200 import host
    env = host.Env(1)
    try:
        env.execute("op.kernel_status")
        assert env.pop_number() == 0
        for text in ("1024 2 io.link.open", "0 0 io.link.wait", "1 io.link.fence", '0 0 4 4 2 "half" io.link.window'):
            with pytest.raises(host.HostError):
                env.execute(text)
            env.clear_stack()
        # the split operators refuse host tensors like every math operator does (no CPU path)
        env.execute('4 4 2 "cpu" "float" op.create "a" !  4 4 2 "cpu" "float" op.create "b" !  4 4 2 "cpu" "float" op.create "c" !')
        with pytest.raises(host.HostError):
            env.execute('"a" @ "b" @ "c" @ op.linear_backward_x')
    finally:
        env.close()
