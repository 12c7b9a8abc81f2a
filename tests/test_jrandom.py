"""The host-side java.util.Random used by sampled generation against the oracle's restatement and the
published first outputs."""
import oracle
from deepj_b200.jrandom import JavaRandom


def test_matches_the_oracle_generator():
    for seed in (0, 7, 42, -3, 2 ** 40 + 5):
        a, b = JavaRandom(seed), oracle.JRandom(seed)
        assert [a.next_float() for _ in range(50)] == [b.next_float() for _ in range(50)]
        assert [a.next_int(256) for _ in range(50)] == [b.next_int(256) for _ in range(50)]
        assert [a.next_int(10) for _ in range(50)] == [b.next_int(10) for _ in range(50)]


def test_documented_first_values():
    assert JavaRandom(42).next_float() == 0.7275636792182922       # new Random(42).nextFloat() = 0.7275637f
    assert [JavaRandom(42).next_int(10)] == [0]                      # new Random(42).nextInt(10) = 0
