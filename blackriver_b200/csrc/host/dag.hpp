// The "words" script machine: a small stack language that scripts tensor allocation and the
// layer mathematics (init.words / train.words).  Grammar and run-time behaviour follow the
// reference machine (blackriver/dag.hpp, blackriver/dag.cpp):
//
//   * separators: white space and the characters ( ) { } (they carry no meaning); [ and ] are
//     tokens; "..." and '...' are strings closed on the same line; ; starts a comment;
//   * literals: numbers (atof when the token has '.' or 'e', else atol), strings, a token that
//     starts with $ is the string of its own spelling, `ture`/`true` -> 1, `false` -> 0,
//     `null` -> "";
//   * %def name ... %end defines a user word (no nesting); user words are inlined where used, so
//     there is no call stack, no recursion and no control flow;
//   * [ a b c ] pushes its items and then their count;
//   * builtins on the current hash table: @ get, ! set (value below name), !! drop,
//     # switch to the popped table index, ## push the current table index;
//   * every use of a native word gets its own NativeWord instance at link time.
//
// Public names (Enviroment, Stack, Hash, Cell, NativeWord, DaG, NWORD_CREATOR_DEFINE_LR) are the
// reference's, so word bindings written against it compile unchanged.
#pragma once

#include <map>
#include <memory>
#include <string>
#include <variant>
#include <vector>

#include "common.hpp"

namespace br {

struct TensorType;
using tensor_t = std::shared_ptr<TensorType>;

struct Cell {
    enum CellType { T_Number, T_String, T_Tensor };
    std::variant<double, std::string, tensor_t> v_;

    Cell() : v_(0.0) {}
    Cell(double n) : v_(n) {}
    Cell(const std::string& s) : v_(s) {}
    Cell(tensor_t t) : v_(std::move(t)) {}

    CellType type() const { return (CellType)v_.index(); }
    bool is_number() const { return v_.index() == 0; }
    bool is_string() const { return v_.index() == 1; }
    bool is_tensor() const { return v_.index() == 2; }
    double as_number() const {
        br_assert(is_number(), "cell is not a number");
        return std::get<0>(v_);
    }
    bool as_boolean() const { return as_number() != 0.0; }
    const std::string& as_string() const {
        br_assert(is_string(), "cell is not a string");
        return std::get<1>(v_);
    }
    tensor_t as_tensor() const {
        br_assert(is_tensor(), "cell is not a tensor");
        return std::get<2>(v_);
    }
};
std::ostream& operator<<(std::ostream& os, const Cell& c);

struct Stack {
    size_t size() const { return data_.size(); }
    void clear() { data_.clear(); }
    Cell& top() {
        need(1);
        return data_.back();
    }
    Cell pop() {
        need(1);
        Cell c = std::move(data_.back());
        data_.pop_back();
        return c;
    }
    void drop() {
        need(1);
        data_.pop_back();
    }
    void dup() { data_.push_back(top()); }
    // ( a b -- a b a b a b ): three copies of the pair, as the reference word does (dag.hpp:107-114)
    void dup2() {
        Cell b = pop(), a = pop();
        for (int i = 0; i < 3; i++) {
            data_.push_back(a);
            data_.push_back(b);
        }
    }
    void swap() {
        need(2);
        std::swap(data_[data_.size() - 1], data_[data_.size() - 2]);
    }
    // ( c b a -- b a c )
    void rot() {
        Cell a = pop(), b = pop(), c = pop();
        data_.push_back(b);
        data_.push_back(a);
        data_.push_back(c);
    }
    double pop_number() { return pop().as_number(); }
    bool pop_boolean() { return pop().as_boolean(); }
    std::string pop_string() { return pop().as_string(); }
    tensor_t pop_tensor() { return pop().as_tensor(); }
    // ( x1 .. xn n -- ) -> {x1 .. xn}
    std::vector<double> pop_number_list() {
        size_t n = (size_t)pop_number();
        std::vector<double> out(n);
        for (size_t i = 0; i < n; i++) out[n - 1 - i] = pop_number();
        return out;
    }
    void push(Cell c) { data_.push_back(std::move(c)); }
    void push_number(double n) { data_.emplace_back(n); }
    void push_string(const std::string& s) { data_.emplace_back(s); }
    void push_tensor(tensor_t t) { data_.emplace_back(std::move(t)); }
    void push_number_list(const std::vector<double>& l) {
        for (double v : l) push_number(v);
        push_number((double)l.size());
    }
    const std::vector<Cell>& cells() const { return data_; }

private:
    void need(size_t n) const { br_assert(data_.size() >= n, "stack underflow"); }
    std::vector<Cell> data_;
};
std::ostream& operator<<(std::ostream& os, const Stack& s);

struct Hash {
    using Item = std::variant<double, std::string, tensor_t>;
    bool has(const std::string& name) const { return map_.count(name) != 0; }
    Item find(const std::string& name) const {
        auto it = map_.find(name);
        if (it == map_.end()) br_panic("no value named '" + name + "' in the current hash");
        return it->second;
    }
    double find_number(const std::string& n) const { return std::get<0>(find(n)); }
    std::string find_string(const std::string& n) const { return std::get<1>(find(n)); }
    tensor_t find_tensor(const std::string& n) const { return std::get<2>(find(n)); }
    void set(const std::string& name, Item item) { map_[name] = std::move(item); }
    void drop(const std::string& name) { map_.erase(name); }
    size_t size() const { return map_.size(); }
    static Cell Item2Cell(const Item& i) { return std::visit([](auto&& v) { return Cell(v); }, i); }
    static Item Cell2Item(const Cell& c) { return c.v_; }

private:
    std::map<std::string, Item> map_;
};

struct Enviroment;
struct NativeWord {
    virtual ~NativeWord() = default;
    virtual void run(Stack& stack) = 0;
};
using NativeCreator = NativeWord*(Enviroment&);

// A linked program: flat instruction list plus the native instances it owns.
struct DaG {
    explicit DaG(Enviroment* env) : env_(env) {}
    DaG(const DaG&) = delete;
    DaG& operator=(const DaG&) = delete;
    ~DaG() {
        for (auto* n : natives_) delete n;
    }
    size_t size() const { return code_.size(); }

private:
    enum OpKind : uint8_t { PushNumber, PushString, Get, Set, Drop, ChangeHash, CurrentHash, Native };
    struct Op {
        OpKind kind;
        double num = 0;
        std::string str;
        size_t idx = 0;
    };
    const Enviroment* env_;
    std::vector<Op> code_;
    std::vector<NativeWord*> natives_;
    friend struct Enviroment;
};

struct Enviroment {
    explicit Enviroment(int hash_num = 1);
    ~Enviroment() = default;

    void insert_native_word(const std::string& name, NativeCreator* fn);
    bool has_word(const std::string& name) const { return natives_.count(name) || users_.count(name); }

    DaG* build(const std::string& txt);   // compile + link; the caller owns the result
    void run(DaG* dag);
    void execute(const std::string& txt);  // build, run once, discard

    Stack& stack() { return stack_; }
    Hash& hash() { return hashes_[target_]; }
    void change(size_t new_hash) {
        if (new_hash >= hashes_.size()) br_panic("hash index out of range");
        target_ = new_hash;
    }
    size_t hashes_current() const { return target_; }
    size_t hashes_num() const { return hashes_.size(); }

    // Optional hook called around every native word (tracing / profiling ranges).
    using TraceFn = void (*)(const char* word, bool begin);
    void set_trace(TraceFn fn) { trace_ = fn; }

private:
    enum ItemKind : uint8_t { INumber, IString, IBuiltin, INative, IUser };
    struct Item {
        ItemKind kind;
        std::string text;
        double num = 0;
    };
    using Word = std::vector<Item>;

    Word compile(const std::string& txt);
    void link(DaG& dag, const Word& w, int depth);
    void load_base_words();

    std::map<std::string, Word> users_;
    std::map<std::string, NativeCreator*> natives_;
    std::vector<std::string> native_names_;  // names of DaG natives are looked up for tracing
    Stack stack_;
    std::vector<Hash> hashes_;
    size_t target_ = 0;
    TraceFn trace_ = nullptr;
    friend struct DaG;
};

#define NWORD_CREATOR_DEFINE_LR(CLS) \
    static NativeWord* creator(Enviroment& env) { return new CLS(); }

}  // namespace br
